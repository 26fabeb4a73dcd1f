"""Loader base class, background prefetching and the device prefetcher's CPU
pass-through (parity: test/single/test_torch.py data-loader tests of
horovod/data/data_loader_base.py)."""
import threading
import time

import pytest
import torch

from horovod_b200.data import AsyncDataLoaderMixin, BaseDataLoader, DevicePrefetcher


class _Loader(BaseDataLoader):
    def __init__(self, n, fail_at=None, delay=0.0):
        self.n, self.fail_at, self.delay = n, fail_at, delay
        self.producer_threads = set()

    def __len__(self):
        return self.n

    def _iterate(self):
        for i in range(self.n):
            self.producer_threads.add(threading.current_thread().name)
            if self.fail_at == i:
                raise ValueError("bad batch %d" % i)
            if self.delay:
                time.sleep(self.delay)
            yield torch.full((2,), float(i))

    def _process_batch(self, batch):
        return batch + 1


class _AsyncLoader(AsyncDataLoaderMixin, _Loader):
    pass


def test_base_loader_processes_batches():
    out = [b.tolist() for b in _Loader(3)]
    assert out == [[1.0, 1.0], [2.0, 2.0], [3.0, 3.0]]


def test_async_loader_runs_in_a_thread_and_keeps_order():
    loader = _AsyncLoader(20, async_loader_queue_size=4)
    for _epoch in range(2):  # restartable
        out = [int(b[0]) for b in loader]
        assert out == list(range(1, 21))
    assert loader.producer_threads == {"hvd-async-data-loader"}
    sync = _AsyncLoader(5, async_loader_queue_size=0)
    assert [int(b[0]) for b in sync] == [1, 2, 3, 4, 5]
    assert threading.current_thread().name in sync.producer_threads


def test_async_loader_propagates_worker_errors_and_can_be_closed():
    loader = _AsyncLoader(10, fail_at=3, async_loader_queue_size=2)
    seen = []
    with pytest.raises(ValueError, match="bad batch 3"):
        for b in loader:
            seen.append(int(b[0]))
    assert seen == [1, 2, 3]
    slow = _AsyncLoader(1000, delay=0.001, async_loader_queue_size=2)
    it = iter(slow)
    next(it)
    slow.close_async_loader()  # must not hang with a full queue
    assert slow._thread is None


def test_device_prefetcher_passthrough_on_cpu():
    batches = [(torch.ones(2) * i, {"y": torch.tensor([i])}) for i in range(4)]
    out = list(DevicePrefetcher(batches, "cpu"))
    assert len(out) == 4 and out[2][1]["y"].item() == 2


@pytest.mark.gpu
def test_device_prefetcher_moves_batches_to_the_gpu():
    batches = [(torch.ones(1 << 16) * i, {"y": torch.tensor([i])}) for i in range(6)]
    got = []
    for x, extra in DevicePrefetcher(batches, "cuda:0"):
        assert x.is_cuda and extra["y"].is_cuda
        got.append((float(x.sum()), int(extra["y"])))
    assert got == [(float(i * (1 << 16)), i) for i in range(6)]
