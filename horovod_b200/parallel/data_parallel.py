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


def shard_sampler(dataset, shuffle=True, seed=0, drop_last=False):
    """A ``DistributedSampler`` for this rank: every rank reads its own shard
    of every epoch (call ``sampler.set_epoch(epoch)`` each epoch)."""
    import torch.utils.data.distributed as dist_data
    return dist_data.DistributedSampler(dataset, num_replicas=hvd.size(), rank=hvd.rank(),
                                        shuffle=shuffle, seed=seed, drop_last=drop_last)


def average_metrics(metrics, name="metrics", process_set=None):
    """Averages a dict of scalars (floats, ints, 0-d or 1-element tensors)
    over the ranks with ONE fused allreduce; returns a dict of floats. What
    the reference's Keras ``MetricAverageCallback`` does at the end of an
    epoch (horovod/_keras/callbacks.py:49-92), for plain training loops."""
    import torch
    keys = sorted(metrics)
    if not keys:
        return {}
    flat = torch.tensor([float(metrics[k]) for k in keys], dtype=torch.float64)
    kwargs = {} if process_set is None else {"process_set": process_set}
    mean = hvd.allreduce(flat, op=hvd.Average, name="%s.%d" % (name, len(keys)), **kwargs)
    return {k: float(v) for k, v in zip(keys, mean.tolist())}


def warmup_lr_scheduler(optimizer, warmup_steps, ranks=None, after=None):
    """Learning-rate schedule for large data-parallel batches: the optimizer is
    created with the rate for the whole job (base rate x ranks); during the
    first ``warmup_steps`` calls of ``scheduler.step()`` the rate grows
    linearly from the single-rank rate to that value ("gradual warm-up",
    the reference's LearningRateWarmupCallback, horovod/_keras/callbacks.py:
    149-187); afterwards ``after(step)`` (default: 1.0) multiplies it.
    Returns a ``torch.optim.lr_scheduler.LambdaLR``."""
    import torch
    n = float(ranks if ranks is not None else hvd.size())
    warmup_steps = max(int(warmup_steps), 0)

    def factor(step):
        if step < warmup_steps:
            return (1.0 + (n - 1.0) * (step + 1) / warmup_steps) / n
        return 1.0 if after is None else float(after(step - warmup_steps))

    base = getattr(optimizer, "_base_optimizer", optimizer)
    return torch.optim.lr_scheduler.LambdaLR(base, lr_lambda=factor)
