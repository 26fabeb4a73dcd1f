"""Sampler that can be repartitioned when the number of workers changes and
that remembers which samples of the current epoch were already consumed.

Parity: horovod/torch/elastic/sampler.py:24-132.
"""
import math
import random

import torch.utils.data.distributed

from horovod_b200.torch.mpi_ops import rank, size


class ElasticSampler(torch.utils.data.Sampler):
    """Partitions the not-yet-processed indices of ``dataset`` among the
    current ranks. Call ``record_batch(batch_idx, batch_size)`` after each
    batch (before ``state.commit()``), and ``set_epoch(epoch)`` at the end of
    each epoch."""

    def __init__(self, dataset, shuffle=True, seed=0):
        self.dataset = dataset
        self.shuffle = shuffle
        self.seed = seed
        self.epoch = 0
        self.processed_indices = set()
        self.num_replicas = 0
        self.rank = 0
        self.remaining_indices = []
        self.num_samples = 0
        self.total_size = 0
        self.reset()

    def set_epoch(self, epoch):
        """Starts a new epoch: clears the processed set and reshuffles."""
        self.epoch = epoch
        self.processed_indices = set()
        self.reset()

    def record_batch(self, batch_idx, batch_size):
        """Marks the indices of batch ``batch_idx`` as processed."""
        self.processed_indices.update(self.get_indices(batch_idx, batch_size))

    def get_indices(self, batch_idx, batch_size):
        start = batch_idx * batch_size
        end = min(start + batch_size, len(self.indices))
        return self.indices[start:end]

    def load_state_dict(self, state_dict):
        self.epoch = state_dict["epoch"]
        self.processed_indices = set(state_dict["processed_indices"])
        self.reset()

    def state_dict(self):
        return dict(epoch=self.epoch, processed_indices=set(self.processed_indices))

    def reset(self):
        """Recomputes this rank's share for the current world size."""
        from horovod_b200.torch.mpi_ops import is_initialized
        self.num_replicas = size() if is_initialized() else 1
        self.rank = rank() if is_initialized() else 0
        self.remaining_indices = [idx for idx in range(len(self.dataset))
                                  if idx not in self.processed_indices]
        self.num_samples = int(math.ceil(len(self.remaining_indices) * 1.0 / self.num_replicas))
        self.total_size = self.num_samples * self.num_replicas

    def __iter__(self):
        self.indices = self.remaining_indices[:]
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(self.indices)
        # Pad so that every rank gets the same number of samples.
        if self.indices:
            while len(self.indices) < self.total_size:
                self.indices += self.indices[:(self.total_size - len(self.indices))]
        self.indices = self.indices[self.rank:self.total_size:self.num_replicas]
        assert len(self.indices) == self.num_samples or not self.remaining_indices
        return iter(self.indices)

    def __len__(self):
        return self.num_samples
