"""Loader base class and asynchronous prefetching.

``BaseDataLoader`` is the contract (``__len__``, ``_iterate``,
``_process_batch``); ``AsyncDataLoaderMixin`` moves ``_iterate`` to a
background thread that feeds a bounded queue, so that batch preparation
overlaps the training step (parity: horovod/data/data_loader_base.py:20-132).

``DevicePrefetcher`` is the GPU half, which the reference leaves to the user:
it keeps one batch ahead in flight on a side CUDA stream, copying from pinned
host memory, and hands each batch to the compute stream without a host
synchronisation (the pattern bench.py uses for its end-to-end number).
"""
import queue
import threading


class BaseDataLoader:
    def __len__(self):
        """Batches per epoch."""
        raise NotImplementedError()

    def _iterate(self):
        """Yields the batches of one epoch."""
        raise NotImplementedError()

    def __iter__(self):
        for batch in self._iterate():
            yield self._process_batch(batch)

    def _process_batch(self, batch):
        """Hook applied to every batch before it reaches the caller."""
        return batch


class AsyncDataLoaderMixin:
    """Put it in front of a loader class:

        class AsyncLoader(AsyncDataLoaderMixin, MyLoader): ...

    ``async_loader_queue_size`` batches are prepared ahead by a daemon thread;
    0 disables the thread. An exception in the worker is re-raised in the
    consumer. ``close_async_loader()`` stops the thread early."""

    _END = object()

    def __init__(self, *args, async_loader_queue_size=64, **kwargs):
        self.async_loader_queue_size = async_loader_queue_size
        super().__init__(*args, **kwargs)
        self._queue = None
        self._thread = None
        self._finished = threading.Event()

    def close_async_loader(self):
        self._finished.set()
        if self._thread is not None:
            # unblock a worker that waits for room in the queue
            try:
                while True:
                    self._queue.get_nowait()
            except queue.Empty:
                pass
            self._thread.join(timeout=10)
            self._thread = None

    def __del__(self):
        try:
            self.close_async_loader()
        except Exception:  # noqa: BLE001 - interpreter shutdown
            pass

    def _put(self, item):
        while not self._finished.is_set():
            try:
                self._queue.put(item, timeout=0.1)
                return True
            except queue.Full:
                continue
        return False

    def _async_worker(self):
        try:
            for batch in self._iterate():
                if not self._put(batch):
                    return
        except Exception as e:  # noqa: BLE001 - delivered to the consumer
            self._put(e)
        self._put(AsyncDataLoaderMixin._END)

    def __iter__(self):
        if self.async_loader_queue_size <= 0:
            for batch in self._iterate():
                yield self._process_batch(batch)
            return
        self.close_async_loader()
        self._finished.clear()
        self._queue = queue.Queue(self.async_loader_queue_size)
        self._thread = threading.Thread(target=self._async_worker, daemon=True,
                                        name="hvd-async-data-loader")
        self._thread.start()
        while True:
            item = self._queue.get()
            if item is AsyncDataLoaderMixin._END:
                break
            if isinstance(item, Exception):
                raise item
            yield self._process_batch(item)
        self._thread.join(timeout=10)
        self._thread = None


class DevicePrefetcher:
    """Wraps an iterable of (nested) CPU tensors and yields them on ``device``,
    one batch ahead: batch i+1 is copied on a side stream (from pinned memory,
    so the copy is asynchronous) while batch i trains. On CPU it is a
    pass-through."""

    def __init__(self, loader, device, pin_memory=True):
        import torch
        self._torch = torch
        self.loader = loader
        self.device = torch.device(device)
        self.pin_memory = pin_memory and self.device.type == "cuda"
        self._stream = torch.cuda.Stream(self.device) if self.device.type == "cuda" else None

    def __len__(self):
        return len(self.loader)

    def _to_device(self, obj):
        torch = self._torch
        if isinstance(obj, torch.Tensor):
            if self.pin_memory and not obj.is_pinned() and obj.device.type == "cpu":
                obj = obj.pin_memory()
            return obj.to(self.device, non_blocking=True)
        if isinstance(obj, (list, tuple)):
            return type(obj)(self._to_device(o) for o in obj)
        if isinstance(obj, dict):
            return {k: self._to_device(v) for k, v in obj.items()}
        return obj

    def _record(self, obj, stream):
        torch = self._torch
        if isinstance(obj, torch.Tensor):
            obj.record_stream(stream)
        elif isinstance(obj, (list, tuple)):
            for o in obj:
                self._record(o, stream)
        elif isinstance(obj, dict):
            for o in obj.values():
                self._record(o, stream)

    def __iter__(self):
        torch = self._torch
        if self._stream is None:
            for batch in self.loader:
                yield batch
            return
        it = iter(self.loader)

        def fetch():
            try:
                batch = next(it)
            except StopIteration:
                return None
            with torch.cuda.stream(self._stream):
                return self._to_device(batch)

        nxt = fetch()
        while nxt is not None:
            current = torch.cuda.current_stream(self.device)
            current.wait_stream(self._stream)
            batch = nxt
            self._record(batch, current)
            nxt = fetch()
            yield batch
