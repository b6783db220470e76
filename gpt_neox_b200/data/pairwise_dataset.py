"""Chosen / rejected pair dataset for DPO and reward-model training (``megatron/data/pairwise_dataset.py``):
document *i* of the ``pos`` corpus is paired with document *i* of the ``neg`` corpus; optional label and
precomputed reference-log-probability side datasets.  Samples are one pair per item (``unpacked``) or pairs
packed until the longer side would overflow (``pack_until_overflow``); ``packed`` is rejected because a pair
must stay aligned."""
from __future__ import annotations

import numpy as np
import torch

from ..utils import print_rank_0


class PairwiseDataset(torch.utils.data.Dataset):
    def __init__(self, name, pos_data_prefix, documents, pos_indexed_dataset, neg_indexed_dataset, num_samples,
                 seq_length, seed, pack_impl="unpacked", build_index_mappings=True, use_shared_fs=True,
                 pos_label_dataset=None, pos_ref_dataset=None, neg_label_dataset=None, neg_ref_dataset=None,
                 allow_chopped=True):
        assert pack_impl != "packed", "Pairwise data cannot be 'packed': pairs must stay aligned"
        self.name, self.seq_length, self.pack_impl, self.allow_chopped = name, seq_length, pack_impl, allow_chopped
        self.pos, self.neg = pos_indexed_dataset, neg_indexed_dataset
        self.pos_label, self.neg_label = pos_label_dataset, neg_label_dataset
        self.pos_ref, self.neg_ref = pos_ref_dataset, neg_ref_dataset
        assert np.min(documents) >= 0 and np.max(documents) < self.pos.sizes.shape[0]
        assert self.pos.sizes.shape[0] == self.neg.sizes.shape[0], "pos and neg corpora must have the same documents"
        rng = np.random.RandomState(seed)
        docs = [d for d in documents if allow_chopped or max(self.pos.sizes[d], self.neg.sizes[d]) <= seq_length + 1]
        n = num_samples if num_samples is not None else len(docs)
        if pack_impl == "unpacked":
            reps = int(np.ceil(n / max(len(docs), 1)))
            order = np.concatenate([rng.permutation(docs) for _ in range(max(reps, 1))])[:n]
            self.groups = [[int(d)] for d in order]
        else:
            self.groups, cur, used = [], [], 0
            while len(self.groups) < n:
                for d in rng.permutation(docs):
                    need = int(max(self.pos.sizes[d], self.neg.sizes[d]))
                    if cur and used + need > seq_length + 1:
                        self.groups.append(cur)
                        cur, used = [], 0
                        if len(self.groups) >= n:
                            break
                    cur.append(int(d))
                    used += need
            self.groups = self.groups[:n]
        print_rank_0(f"    {name}: {len(self.groups)} pairwise samples")

    def __len__(self):
        return len(self.groups)

    def _cat(self, ds, docs, pad, dtype):
        if ds is None:
            return None
        arr = np.concatenate([np.asarray(ds.get(d)) for d in docs]).astype(dtype)
        L = self.seq_length + 1
        if len(arr) < L:
            arr = np.pad(arr, (0, L - len(arr)), constant_values=pad)
        return arr[:L]

    def __getitem__(self, idx):
        docs = self.groups[idx % len(self.groups)]
        out = {"pos": self._cat(self.pos, docs, 0, np.int64), "neg": self._cat(self.neg, docs, 0, np.int64)}
        if self.pos_label is not None:
            out["pos_label"] = self._cat(self.pos_label, docs, -100, np.int64)
            out["neg_label"] = self._cat(self.neg_label, docs, -100, np.int64)
        if self.pos_ref is not None:
            out["pos_ref"] = self._cat(self.pos_ref, docs, 0, np.float32)
            out["neg_ref"] = self._cat(self.neg_ref, docs, 0, np.float32)
        return out
