"""Data parallelism in two calls.

    model, optimizer = data_parallel_setup(model, optimizer)

wraps ``optimizer`` in ``hvd.DistributedOptimizer`` (gradients averaged over
all ranks, in place in symmetric memory on one NVSwitch box) and starts every
rank from rank 0's weights and optimizer state, which is the sequence of the
reference's examples (examples/pytorch/pytorch_synthetic_benchmark.py:59-72).
"""
import horovod_b200.torch as hvd
from horovod_b200.torch import DistributedOptimizer, SyncBatchNorm  # noqa: F401


def broadcast_model_and_optimizer(model, optimizer, root_rank=0):
    """Every rank continues from ``root_rank``'s parameters, buffers and
    optimizer state."""
    hvd.broadcast_parameters(model.state_dict(), root_rank=root_rank)
    hvd.broadcast_optimizer_state(optimizer, root_rank=root_rank)


def data_parallel_setup(model, optimizer, compression=None, symmetric_gradients=None,
                        root_rank=0, **optimizer_kwargs):
    """Returns ``(model, distributed_optimizer)`` ready for a training loop.
    ``hvd.init()`` must have been called; the model must already be on its
    device."""
    kwargs = dict(optimizer_kwargs)
    if compression is not None:
        kwargs["compression"] = compression
    wrapped = hvd.DistributedOptimizer(optimizer, named_parameters=model.named_parameters(),
                                       symmetric_gradients=symmetric_gradients, **kwargs)
    broadcast_model_and_optimizer(model, wrapped, root_rank)
    return model, wrapped
