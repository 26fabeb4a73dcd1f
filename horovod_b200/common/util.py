"""Small helpers shared by the Python layers.

Parity: horovod/common/util.py:33-267 (split_list, num_rank_is_power_2,
average/op back-compat handling, build-feature queries).
"""
import os
import warnings


def split_list(items, num_parts):
    """Splits ``items`` into ``num_parts`` contiguous chunks whose sizes
    differ by at most one (earlier chunks are the longer ones)."""
    base, extra = divmod(len(items), num_parts)
    out, pos = [], 0
    for i in range(num_parts):
        n = base + (1 if i < extra else 0)
        out.append(items[pos:pos + n])
        pos += n
    return out


def num_rank_is_power_2(num_rank):
    return num_rank != 0 and (num_rank & (num_rank - 1)) == 0


def get_average_backwards_compatibility_fun(reduce_ops):
    """Returns handle_average_backwards_compatibility(op, average), which
    resolves the deprecated ``average=`` flag against ``op=``."""

    def impl(op, average):
        if op is not None:
            if average is not None:
                raise ValueError("The op parameter supersedes average. "
                                 "Please provide only one of them.")
            return op
        if average is not None:
            warnings.warn("Parameter `average` has been replaced with `op` "
                          "and will be removed", DeprecationWarning)
            return reduce_ops.Average if average else reduce_ops.Sum
        return reduce_ops.Average

    return impl


def env_flag(name, default=False):
    v = os.environ.get(name)
    if v is None or v == "":
        return default
    return v.strip().lower() in ("1", "true", "yes", "on")


def is_iterable(x):
    try:
        iter(x)
    except TypeError:
        return False
    return True
