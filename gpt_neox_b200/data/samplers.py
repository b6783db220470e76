"""Batch samplers for data-parallel training (capabilities of ``megatron/data/samplers.py:24-169``).

``DistributedBatchSampler`` cuts the index stream of an underlying sampler into *global* batches and hands each
data-parallel rank its share of every batch: a contiguous block of ``batch_size // world_size`` indices by default,
every ``world_size``-th index when ``interleave`` is set.  ``start_iter`` makes a resumed run skip the global
batches it has already consumed; ``wrap_last`` carries an incomplete final batch over into the next pass instead
of emitting a short one.  ``RandomSampler`` draws a fresh permutation per epoch, seeded by the epoch number, so
every rank (and every restart) sees the same order.
"""
from __future__ import annotations

import itertools

import torch
from torch.utils import data


class RandomSampler(data.Sampler):
    """Permutation (or draws with replacement) of ``range(len(data_source))``; ``set_epoch(e)`` seeds it with ``e``."""

    def __init__(self, data_source, replacement=False, num_samples=None):
        if num_samples is not None and not replacement:
            raise ValueError("num_samples only makes sense with replacement=True (a permutation has a fixed length)")
        count = len(data_source) if num_samples is None else num_samples
        if not isinstance(count, int) or count <= 0:
            raise ValueError(f"the sampler needs a positive number of samples, got {count}")
        self.data_source, self.replacement, self._count = data_source, replacement, count
        self.epoch = -1

    @property
    def num_samples(self):
        return self._count

    def set_epoch(self, epoch):
        self.epoch = epoch

    def _generator(self):
        g = torch.Generator()
        if self.epoch >= 0:
            g.manual_seed(self.epoch)
        return g

    def __iter__(self):
        population = len(self.data_source)
        if self.replacement:
            draws = torch.randint(population, (self._count,), generator=self._generator(), dtype=torch.int64)
        else:
            draws = torch.randperm(population, generator=self._generator())
        yield from draws.tolist()

    def __len__(self):
        return self._count


class DistributedBatchSampler(data.BatchSampler):
    """This rank's slice of each global batch (see module docstring)."""

    def __init__(self, sampler, batch_size, drop_last, rank=-1, world_size=2, wrap_last=False, interleave=False):
        super().__init__(sampler, batch_size, drop_last)
        if not 0 <= rank < world_size:
            raise ValueError(f"rank {rank} is not a member of a data-parallel group of size {world_size}")
        if batch_size % world_size:
            raise ValueError(f"global batch {batch_size} does not divide over {world_size} ranks")
        self.rank, self.world_size = rank, world_size
        self.wrap_last, self.interleave = wrap_last, interleave
        self.start_iter = 0      # global batches to skip on the next pass (resume)
        self._carry = 0          # indices at the head of the next pass already served by a wrapped batch

    def _mine(self, global_batch):
        if self.interleave:
            return global_batch[self.rank::self.world_size]
        share = self.batch_size // self.world_size
        return global_batch[self.rank * share:(self.rank + 1) * share]

    def __iter__(self):
        stream = itertools.islice(iter(self.sampler), self._carry, None)
        self._carry = 0
        skip, self.start_iter = self.start_iter, 0
        for number in itertools.count():
            chunk = list(itertools.islice(stream, self.batch_size))
            if len(chunk) < self.batch_size:
                break
            if number >= skip:
                yield self._mine(chunk)
        if chunk and not self.drop_last:
            if self.wrap_last:
                # complete the batch from the head of the sampler; the next pass starts after the borrowed part
                missing = self.batch_size - len(chunk)
                chunk += list(itertools.islice(iter(self.sampler), missing))
                self._carry = missing
            yield self._mine(chunk)
