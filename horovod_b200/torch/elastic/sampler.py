"""Sampler for elastic training: it splits the samples of an epoch that have
not been consumed yet among however many ranks there are right now, so an
epoch can continue across a change of membership without repeating data.

The training loop calls ``record_batch(batch_idx, batch_size)`` after every
batch (before ``state.commit()``) and ``set_epoch(epoch)`` when an epoch ends;
``hvd.elastic.TorchState(sampler=...)`` merges the consumed sets of all ranks
at every sync and calls ``reset()``.

API and semantics follow horovod/torch/elastic/sampler.py:24-132 (every rank
draws the same number of samples; the tail is padded by repeating the head).
"""
import random

import torch.utils.data

from horovod_b200.torch.mpi_ops import is_initialized, rank, size


class ElasticSampler(torch.utils.data.Sampler):
    def __init__(self, dataset, shuffle=True, seed=0):
        self.dataset = dataset
        self.shuffle = shuffle
        self.seed = seed
        self.epoch = 0
        self.processed_indices = set()
        self.indices = []
        self.reset()

    # ---- bookkeeping the training loop drives --------------------------------
    def set_epoch(self, epoch):
        """A new epoch: nothing is consumed yet, and the shuffle changes."""
        self.epoch = epoch
        self.processed_indices = set()
        self.reset()

    def get_indices(self, batch_idx, batch_size):
        """Dataset indices this rank used for batch ``batch_idx`` of the
        current pass."""
        first = batch_idx * batch_size
        return self.indices[first:first + batch_size]

    def record_batch(self, batch_idx, batch_size):
        self.processed_indices.update(self.get_indices(batch_idx, batch_size))

    def state_dict(self):
        return {"epoch": self.epoch, "processed_indices": set(self.processed_indices)}

    def load_state_dict(self, state_dict):
        self.epoch = state_dict["epoch"]
        self.processed_indices = set(state_dict["processed_indices"])
        self.reset()

    # ---- partitioning ---------------------------------------------------------
    def reset(self):
        """Re-reads the world size and recomputes what is left to share out."""
        self.num_replicas, self.rank = (size(), rank()) if is_initialized() else (1, 0)
        done = self.processed_indices
        self.remaining_indices = [i for i in range(len(self.dataset)) if i not in done]
        # ceil(remaining / replicas) samples per rank
        self.num_samples = -(-len(self.remaining_indices) // self.num_replicas)
        self.total_size = self.num_samples * self.num_replicas

    def __iter__(self):
        order = list(self.remaining_indices)
        if self.shuffle:
            random.Random(self.seed + self.epoch).shuffle(order)
        # Every rank must draw the same number of samples: wrap around.
        short = self.total_size - len(order)
        if order and short > 0:
            order += [order[i % len(order)] for i in range(short)]
        self.indices = order[self.rank:self.total_size:self.num_replicas]
        return iter(self.indices)

    def __len__(self):
        return self.num_samples
