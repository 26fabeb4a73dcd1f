"""Operators of the framework: the collectives (re-exported from
horovod_b200.torch) and the model-side fused kernels."""
from horovod_b200.ops.batch_norm import BatchNormAct2d, batch_norm_act  # noqa: F401


def __getattr__(name):
    # Collectives live in horovod_b200.torch; resolve them lazily so that
    # importing the model-side ops does not initialise anything.
    import horovod_b200.torch as hvd
    if name in ("allreduce", "allreduce_", "grouped_allreduce", "grouped_allreduce_",
                "allgather", "broadcast", "broadcast_", "alltoall", "reducescatter",
                "symmetric_empty"):
        return getattr(hvd, name)
    raise AttributeError(name)
