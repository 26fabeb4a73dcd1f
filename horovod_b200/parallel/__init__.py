"""Data-parallel building blocks (the parallelism strategy the reference
offers): wrapped optimizer, state broadcast, synchronized batch norm and
process sets, gathered in one namespace."""
from horovod_b200.parallel.data_parallel import (  # noqa: F401
    DistributedOptimizer, SyncBatchNorm, average_metrics, broadcast_model_and_optimizer,
    data_parallel_setup, shard_sampler, warmup_lr_scheduler)
