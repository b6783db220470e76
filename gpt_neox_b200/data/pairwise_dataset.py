"""Chosen / rejected pair dataset for DPO and reward-model training (``megatron/data/pairwise_dataset.py``):
document *i* of the ``pos`` corpus is paired with document *i* of the ``neg`` corpus; optional label and
precomputed reference-log-probability side datasets.  Samples are one pair per item (``unpacked``) or pairs
packed until the longer side would overflow (``pack_until_overflow``); ``packed`` is rejected because a pair
must stay aligned.  The sample index (which documents make up sample *i*) is cached as ``.npy`` files next to the
``pos`` corpus, like the index maps of the language-model dataset."""
from __future__ import annotations

import os
import time

import numpy as np
import torch

from ..utils import print_rank_0
from .gpt2_dataset import _io_barrier, _is_builder


def _build_groups(docs, pos_sizes, neg_sizes, n, seq_length, pack_impl, rng):
    """Documents of every sample as a flat array plus sample boundaries (sample i = doc_idx[start[i]:start[i + 1]])."""
    if pack_impl == "unpacked":
        reps = int(np.ceil(n / max(len(docs), 1)))
        order = np.concatenate([rng.permutation(docs) for _ in range(max(reps, 1))])[:n]
        return order.astype(np.int64), np.arange(len(order) + 1, dtype=np.int64)
    doc_idx, starts, used = [], [0], 0
    while len(starts) <= n:
        for d in rng.permutation(docs):
            need = int(max(pos_sizes[d], neg_sizes[d]))
            if len(doc_idx) > starts[-1] and used + need > seq_length + 1:
                starts.append(len(doc_idx))
                used = 0
                if len(starts) > n:
                    break
            doc_idx.append(int(d))
            used += need
    return np.asarray(doc_idx[:starts[n]], dtype=np.int64), np.asarray(starts[:n + 1], dtype=np.int64)


class PairwiseDataset(torch.utils.data.Dataset):
    def __init__(self, name, pos_data_prefix, documents, pos_indexed_dataset, neg_indexed_dataset, num_samples,
                 seq_length, seed, pack_impl="unpacked", build_index_mappings=True, use_shared_fs=True,
                 pos_label_dataset=None, pos_ref_dataset=None, neg_label_dataset=None, neg_ref_dataset=None,
                 allow_chopped=True):
        assert pack_impl != "packed", "Pairwise data cannot be 'packed': pairs must stay aligned"
        self.name, self.seq_length, self.pack_impl, self.allow_chopped = name, seq_length, pack_impl, allow_chopped
        self.pos, self.neg = pos_indexed_dataset, neg_indexed_dataset
        self.indexed_dataset = self.pos            # what the weighting by number of documents counts
        self.pos_label, self.neg_label = pos_label_dataset, neg_label_dataset
        self.pos_ref, self.neg_ref = pos_ref_dataset, neg_ref_dataset
        assert np.min(documents) >= 0 and np.max(documents) < self.pos.sizes.shape[0]
        assert self.pos.sizes.shape[0] == self.neg.sizes.shape[0], "pos and neg corpora must have the same documents"
        self.doc_idx, self.starts = np.zeros(0, dtype=np.int64), np.zeros(1, dtype=np.int64)
        if not build_index_mappings:               # a first pass that only wants the document counts
            return
        docs = [d for d in documents if allow_chopped or max(self.pos.sizes[d], self.neg.sizes[d]) <= seq_length + 1]
        n = num_samples if num_samples is not None else len(docs)
        # the index is cached next to the data, keyed by everything it depends on; one rank builds, all load
        base = f"{pos_data_prefix}_{name}_pairmap_{n}ns_{seq_length}sl_{seed}s_{pack_impl}pi" + \
            ("_ac" if allow_chopped else "")
        f_doc, f_start = base + "_doc_idx.npy", base + "_sample_idx.npy"
        cache = os.path.isdir(os.path.dirname(os.path.abspath(str(pos_data_prefix)))) and \
            os.path.isfile(str(pos_data_prefix) + ".idx")
        if not cache:                              # in-memory corpora (tests, synthetic pairs): nothing to put it beside
            self.doc_idx, self.starts = _build_groups(docs, self.pos.sizes, self.neg.sizes, n, seq_length, pack_impl,
                                                      np.random.RandomState(seed))
        else:
            if _is_builder(use_shared_fs) and not (os.path.isfile(f_doc) and os.path.isfile(f_start)):
                print_rank_0(" > WARNING: could not find pairwise index map files, building the indices ...")
                t0 = time.time()
                doc_idx, starts = _build_groups(docs, self.pos.sizes, self.neg.sizes, n, seq_length, pack_impl,
                                                np.random.RandomState(seed))
                np.save(f_doc, doc_idx, allow_pickle=True)
                np.save(f_start, starts, allow_pickle=True)
                print_rank_0(f" > elapsed time to build and save pairwise index mappings (seconds): "
                             f"{time.time() - t0:4f}")
            _io_barrier()
            self.doc_idx = np.load(f_doc, allow_pickle=True, mmap_mode="r")
            self.starts = np.load(f_start, allow_pickle=True, mmap_mode="r")
        print_rank_0(f"    {name}: {len(self)} pairwise samples")

    @property
    def groups(self):
        """The documents of every sample, as lists."""
        return [[int(d) for d in self.doc_idx[self.starts[i]:self.starts[i + 1]]] for i in range(len(self))]

    def __len__(self):
        return len(self.starts) - 1

    def _cat(self, ds, docs, pad, dtype):
        if ds is None:
            return None
        arr = np.concatenate([np.asarray(ds.get(d)) for d in docs]).astype(dtype)
        L = self.seq_length + 1
        if len(arr) < L:
            arr = np.pad(arr, (0, L - len(arr)), constant_values=pad)
        return arr[:L]

    def __getitem__(self, idx):
        i = idx % len(self)
        docs = [int(d) for d in self.doc_idx[self.starts[i]:self.starts[i + 1]]]
        out = {"pos": self._cat(self.pos, docs, 0, np.int64), "neg": self._cat(self.neg, docs, 0, np.int64)}
        if self.pos_label is not None:
            out["pos_label"] = self._cat(self.pos_label, docs, -100, np.int64)
            out["neg_label"] = self._cat(self.neg_label, docs, -100, np.int64)
        if self.pos_ref is not None:
            out["pos_ref"] = self._cat(self.pos_ref, docs, 0, np.float32)
            out["neg_ref"] = self._cat(self.neg_ref, docs, 0, np.float32)
        return out
