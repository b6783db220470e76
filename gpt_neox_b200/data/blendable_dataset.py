"""Weighted mixture of datasets (``megatron/data/blendable_dataset.py:29-82``): sample *i* of the blend is
sample ``dataset_sample_index[i]`` of dataset ``dataset_index[i]``, with the interleaving computed by the
C++ greedy-deficit builder."""
from __future__ import annotations

import time

import numpy as np
import torch

from ..utils import print_rank_0
from . import helpers


class BlendableDataset(torch.utils.data.Dataset):
    def __init__(self, datasets, weights):
        self.datasets = datasets
        n = len(datasets)
        assert n == len(weights)
        self.size = sum(len(d) for d in datasets)
        w = np.array(weights, dtype=np.float64)
        assert w.sum() > 0.0
        w /= w.sum()
        assert n < 255
        t0 = time.time()
        self.dataset_index, self.dataset_sample_index = helpers.build_blending_indices(w, self.size)
        print_rank_0(f"> elapsed time for building blendable dataset indices: {time.time() - t0:.2f} (sec)")

    def __len__(self):
        return self.size

    def __getitem__(self, idx):
        try:
            return self.datasets[self.dataset_index[idx]][int(self.dataset_sample_index[idx])]
        except IndexError:
            new_idx = idx % len(self)
            print(f"WARNING: Got index out of bounds error with index {idx} - taking modulo of index instead ({new_idx})")
            return self[new_idx]
