"""Introspection helpers: GPU topology, which device path is active, per-op
device timings, kernel launch counts and phase traces."""


def _ext():
    from horovod_b200 import _C
    return _C


def gpu_topology():
    """Devices, SM counts and NVLink/peer connectivity of this box (NVML)."""
    return _ext().gpu_topology()


def gpu_backend():
    """``"symm ranks=N nvls=0|1 ..."`` or ``"nccl"``: the active device path."""
    return _ext().gpu_backend()


def op_timings():
    """Drains the per-response device timings collected with
    HOROVOD_GPU_OP_TIMING=1: tuples (type, bytes, tensors, microseconds)."""
    return _ext().gpu_op_stats()


def response_paths():
    """``{"symm": n, "nccl": m}``: how many device responses this process has
    executed with the symmetric-memory kernels and on the NCCL path (Min /
    Max / Product, bool and 16-bit integer reductions, process sets with id 8
    or more, jobs that span hosts). Read it before and after a call to see
    which path that call took."""
    return dict(_ext().gpu_response_paths())


def kernel_launch_count():
    """Kernels of this library launched so far in this process."""
    return _ext().kernel_launch_count()


def kernel_trace():
    """Device timestamps (ns) at the phase boundaries of the last traced
    allreduce kernel (HOROVOD_KERNEL_TRACE=1)."""
    return _ext().kernel_trace()
