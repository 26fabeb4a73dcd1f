"""Elastic training for PyTorch: ``@hvd.elastic.run`` plus TorchState and
ElasticSampler.

Parity: horovod/torch/elastic/__init__.py:23-48.
"""
from horovod_b200.common.elastic import ObjectState, run_fn
from horovod_b200.torch.elastic.sampler import ElasticSampler
from horovod_b200.torch.elastic.state import TorchState
from horovod_b200.torch.mpi_ops import init, shutdown


def run(func):
    """Decorator for the training function ``func(state, ...)``. On a failed
    collective the state is restored to the last commit; on a host change it
    is kept; either way the runtime is re-initialised with the new set of
    workers, state is synced from rank 0 and ``func`` is called again."""
    return run_fn(func, _reset)


def _reset():
    shutdown()
    init()
