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


# ---- build and environment queries (horovod/common/util.py:33-211, 251-259) ---

def get_ext_suffix():
    """File name suffix of extension modules of this interpreter."""
    import sysconfig
    return sysconfig.get_config_var("EXT_SUFFIX") or ".so"


def get_extension_full_path(pkg_path, *args):
    """Path of the extension module ``args`` joined, next to ``pkg_path``: the
    plain ``name.so`` this repository builds in tree, or the name with the
    interpreter's suffix when that file exists instead."""
    directory = os.path.dirname(os.path.abspath(pkg_path))
    base = os.path.join(directory, *args)
    for candidate in (base + ".so", base + get_ext_suffix()):
        if os.path.exists(candidate):
            return candidate
    return base + ".so"


def check_extension(ext_name, ext_env_var, pkg_path, *args):
    """Raises ImportError with a build hint when the native extension of
    ``ext_name`` is missing (horovod/common/util.py:53-61)."""
    full_path = get_extension_full_path(pkg_path, *args)
    if not os.path.exists(full_path):
        raise ImportError(
            "Extension %s has not been built: %s not found. Run `python horovod_b200/build_ext.py` "
            "(or reinstall with %s=1)." % (ext_name, full_path, ext_env_var))


def extension_available(ext_base_name="torch", verbose=False):
    """Whether the native extension can be loaded (the reference probes this
    in a child process; here importing it has no side effects)."""
    try:
        from horovod_b200 import _C  # noqa: F401
        return True
    except ImportError as e:
        if verbose:
            print("Extension %s is not available: %s" % (ext_base_name, e))
        return False


def gpu_available(ext_base_name="torch", verbose=False):
    """Whether the extension was built with device support and a GPU is visible."""
    if not extension_available(ext_base_name, verbose):
        return False
    try:
        import torch
        return bool(torch.cuda.is_available())
    except ImportError:
        return False


def _build_query(name):
    def query(verbose=False):
        from horovod_b200.common.basics import HorovodBasics
        return bool(getattr(HorovodBasics(), name)())
    query.__name__ = name
    query.__doc__ = "Build feature query (horovod/common/util.py:137-186)."
    return query


mpi_built = _build_query("mpi_built")
gloo_built = _build_query("gloo_built")
nccl_built = _build_query("nccl_built")
ddl_built = _build_query("ddl_built")
ccl_built = _build_query("ccl_built")


class env:  # noqa: N801 - lower case as in the reference
    """Context manager that sets environment variables and restores the old
    values afterwards (horovod/common/util.py:188-211)."""

    def __init__(self, **kwargs):
        self._new = {k: str(v) for k, v in kwargs.items()}
        self._old = {}

    def __enter__(self):
        for k, v in self._new.items():
            self._old[k] = os.environ.get(k)
            os.environ[k] = v
        return self

    def __exit__(self, *exc):
        for k, old in self._old.items():
            if old is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = old
        return False


def check_installed_version(name, version, exception=None):
    """Warns when the framework this extension was built against differs from
    the one imported now."""
    from horovod_b200 import __dict__ as pkg
    built = pkg.get("_built_with", {}).get(name)
    if built is not None and built != version:
        warnings.warn("horovod_b200 was built against %s %s but %s %s is imported; "
                      "rebuild the extension." % (name, built, name, version))
    elif exception is not None and built is None:
        pass  # nothing recorded at build time: nothing to compare
