"""Data-loading helpers: a loader base class, a background-thread prefetch
mixin, and a pinned-memory device prefetcher for the training loop."""
from horovod_b200.data.data_loader_base import (  # noqa: F401
    AsyncDataLoaderMixin, BaseDataLoader, DevicePrefetcher)
