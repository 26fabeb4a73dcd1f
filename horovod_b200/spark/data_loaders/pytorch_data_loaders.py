"""Epoch-wise loaders over ``ParquetShardReader``.

``ParquetDataLoader`` yields a fixed number of batches per epoch (the same on
every rank) from the rank's endless reader, which goes on where the last
epoch stopped; ``AsyncParquetDataLoader`` prepares them ahead of the training
loop on a background thread. Batches are dicts of numpy arrays, or what
``to_tensors`` makes of them.

Parity: horovod/spark/data_loaders/pytorch_data_loaders.py (PytorchDataLoader,
PytorchAsyncDataLoader and their in-memory variants, which wrap a Petastorm
reader); here ``cache=True`` on the reader is the in-memory variant.
"""
from horovod_b200.data.data_loader_base import AsyncDataLoaderMixin, BaseDataLoader
from horovod_b200.spark.common.dataset import ParquetShardReader, steps_per_epoch


class ParquetDataLoader(BaseDataLoader):
    def __init__(self, store, path, columns, batch_size, total_rows, rank=0, size=1, shuffle=True,
                 seed=0, cache=False, transform=None, limit_step_per_epoch=None, to_tensors=None):
        self._reader = ParquetShardReader(store, path, columns, batch_size, rank=rank, size=size,
                                          shuffle=shuffle, seed=seed, cache=cache,
                                          transform=transform)
        self._batches = iter(self._reader)
        self._steps = steps_per_epoch(total_rows, batch_size, size, limit_step_per_epoch)
        self._to_tensors = to_tensors

    def __len__(self):
        return self._steps

    def _iterate(self):
        for _ in range(self._steps):
            yield next(self._batches)

    def _process_batch(self, batch):
        return self._to_tensors(batch) if self._to_tensors else batch


class AsyncParquetDataLoader(AsyncDataLoaderMixin, ParquetDataLoader):
    """``async_loader_queue_size`` batches ahead (0 reads in the training
    thread)."""
