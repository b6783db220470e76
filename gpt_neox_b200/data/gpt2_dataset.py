"""Sample-level view of an indexed token dataset (behaviour of ``megatron/data/gpt2_dataset.py``).

Three index arrays, cached next to the data as ``.npy`` files keyed by name / number of samples /
sequence length / seed / packing mode:

* ``doc_idx``     document order, epochs concatenated, each epoch shuffled (the last epoch is shuffled
                  separately when it would be used only partially);
* ``sample_idx``  ``[n+1, 2]`` (position in doc_idx, token offset): sample *i* spans from row *i* to row *i+1*;
* ``shuffle_idx`` permutation of the samples.

``pack_impl``: ``packed`` (documents concatenated, every sample has exactly ``seq_length+1`` tokens),
``pack_until_overflow`` (whole documents are packed until the next would overflow), ``unpacked`` (one
document per sample, padded).  Optional label / reward / reference-logprob side datasets are sliced
with the same indices; padding is ``-100`` for labels.
"""
from __future__ import annotations

import os
import time

import numpy as np
import torch
import torch.distributed as dist

from ..utils import print_rank_0
from . import helpers


class GPT2Dataset(torch.utils.data.Dataset):
    def __init__(self, name, data_prefix, documents, indexed_dataset, num_samples, num_epochs, seq_length, seed,
                 pack_impl="packed", allow_chopped=True, build_index_mappings=True, use_shared_fs=True,
                 label_dataset=None, reward_dataset=None, ref_dataset=None):
        self.name = name
        self.pack_impl = pack_impl
        self.allow_chopped = allow_chopped
        self.indexed_dataset = indexed_dataset
        self.label_dataset, self.reward_dataset, self.ref_dataset = label_dataset, reward_dataset, ref_dataset
        self.seq_length = seq_length
        assert self.reward_dataset is None or pack_impl == "unpacked", "Reward dataset only compatible with unpacked mode"
        assert np.min(documents) >= 0
        assert np.max(documents) < indexed_dataset.sizes.shape[0]
        if build_index_mappings:
            self.doc_idx, self.sample_idx, self.shuffle_idx = _build_index_mappings(
                name, data_prefix, documents, indexed_dataset.sizes, label_dataset, num_samples, num_epochs,
                seq_length, seed, pack_impl, use_shared_fs=use_shared_fs, allow_chopped=allow_chopped)
            self.shuffle_idx_len = self.shuffle_idx.shape[0] - 1
            self.sample_idx_len = self.sample_idx.shape[0] - 1
            if self.shuffle_idx_len != self.sample_idx_len - 1:
                print(f"WARNING: shuffle index length ({self.shuffle_idx_len}) is not equal to sample index length "
                      f"({self.sample_idx_len})")

    def __len__(self):
        return min(self.shuffle_idx_len, self.sample_idx_len)

    def _side(self):
        ds = [self.indexed_dataset]
        rw = ref = -1
        if self.label_dataset is not None:
            ds.append(self.label_dataset)
        if self.reward_dataset is not None:
            rw = len(ds)
            ds.append(self.reward_dataset)
        if self.ref_dataset is not None:
            ref = len(ds)
            ds.append(self.ref_dataset)
        return ds, rw, ref

    def __getitem__(self, idx):
        try:
            idx = self.shuffle_idx[idx]
            f_doc, f_off = int(self.sample_idx[idx][0]), int(self.sample_idx[idx][1])
            l_doc, l_off = int(self.sample_idx[idx + 1][0]), int(self.sample_idx[idx + 1][1])
            datasets, rw_i, ref_i = self._side()
            samples, sample_lengths = [], []
            pad_for = lambda n: -100 if (n == 1 and self.label_dataset is not None) else 0
            for n, ds in enumerate(datasets):
                if n == rw_i:
                    rw = ds.get(self.doc_idx[f_doc])
                    samples.append(np.array([rw[0] for _ in range(len(samples[-1]))]))
                    continue
                if f_doc == l_doc:
                    samples.append(ds.get(self.doc_idx[f_doc], offset=f_off, length=l_off - f_off + 1))
                elif self.pack_impl != "unpacked":
                    parts = [ds.get(self.doc_idx[f_doc], offset=f_off)]
                    for i in range(f_doc + 1, l_doc):
                        parts.append(ds.get(self.doc_idx[i]))
                    parts.append(ds.get(self.doc_idx[l_doc], length=l_off + 1))
                    samples.append(np.concatenate(parts))
                else:
                    # one document per sample: take the whole document, cut / pad below
                    samples.append(ds.get(self.doc_idx[f_doc], offset=0))
            for n in range(len(samples)):
                pad = pad_for(n) if n != ref_i and n != rw_i else 0
                s = samples[n]
                if len(s) < self.seq_length + 1:
                    s = np.pad(s, (0, self.seq_length + 1 - len(s)), mode="constant", constant_values=pad)
                elif len(s) > self.seq_length + 1:
                    s = s[: self.seq_length + 1]
                samples[n] = s
            ret = {"text": np.array(samples[0], dtype=np.int64)}
            nxt = 1
            if self.label_dataset is not None:
                ret["label"] = np.array(samples[nxt], dtype=np.int64)
                nxt += 1
            if self.reward_dataset is not None:
                ret["reward"] = np.array(samples[rw_i], dtype=np.float32)
            if self.ref_dataset is not None:
                ret["ref"] = np.array(samples[ref_i], dtype=np.float32)
            return ret
        except IndexError:
            new_idx = idx % len(self)
            print(f"WARNING: Got index out of bounds error with index {idx} - taking modulo of index instead ({new_idx})")
            return self[new_idx]


def _num_tokens(documents, sizes):
    return int(np.sum(sizes[documents]))


def _num_epochs(tokens_per_epoch, seq_length, num_samples):
    epochs, total = 0, 0
    while True:
        epochs += 1
        total += tokens_per_epoch
        if ((total - 1) // seq_length) >= num_samples:
            return epochs


def _build_doc_idx(documents, num_epochs, np_rng):
    doc_idx = np.mgrid[0:num_epochs, 0:len(documents)][1]
    doc_idx[:] = documents
    doc_idx = doc_idx.reshape(-1).astype(np.int32)
    np_rng.shuffle(doc_idx)
    return doc_idx


def _build_shuffle_idx(size, np_rng):
    dtype_ = np.uint32 if size < (np.iinfo(np.uint32).max - 1) else np.int64
    shuffle_idx = np.arange(start=0, stop=size, step=1, dtype=dtype_)
    np_rng.shuffle(shuffle_idx)
    return shuffle_idx


def _io_barrier():
    """Wait for the rank that builds the index files.  Only the ranks that load data come here (tensor-parallel rank
    0 of the first and last pipeline stages), so the barrier runs over their group, not over the world."""
    if not (dist.is_available() and dist.is_initialized()):
        return
    from ..parallel import mpu
    if mpu.model_parallel_is_initialized():
        group = mpu.get_io_parallel_group()
        if group is not None:
            dist.barrier(group=group)
        return
    dist.barrier()


def _is_builder(use_shared_fs):
    if not (dist.is_available() and dist.is_initialized()):
        return True
    if not use_shared_fs:
        return int(os.environ.get("LOCAL_RANK", "0")) == 0
    return dist.get_rank() == 0


def _build_index_mappings(name, data_prefix, documents, sizes, label_dataset, num_samples, num_epochs, seq_length,
                          seed, packing_impl, use_shared_fs=True, allow_chopped=True):
    tokens_per_epoch = _num_tokens(documents, sizes)
    if not num_epochs:
        num_epochs = _num_epochs(tokens_per_epoch, seq_length, num_samples)
    np_rng = np.random.RandomState(seed=seed)
    base = f"{data_prefix}_{name}_indexmap_{num_samples}ns_{seq_length}sl_{seed}s_{packing_impl}pi"
    if allow_chopped:
        base += "_ac"
    f_doc, f_sample, f_shuffle = base + "_doc_idx.npy", base + "_sample_idx.npy", base + "_shuffle_idx.npy"
    if _is_builder(use_shared_fs) and not all(os.path.isfile(f) for f in (f_doc, f_sample, f_shuffle)):
        print_rank_0(" > WARNING: could not find index map files, building the indices on rank 0 ...")
        t0 = time.time()
        if packing_impl == "packed":
            doc_idx = _build_doc_idx(documents, num_epochs, np_rng)
            sample_idx = helpers.build_sample_idx(np.asarray(sizes, dtype=np.int32), doc_idx, seq_length, num_epochs,
                                                  tokens_per_epoch)
            shuffle_idx = _build_shuffle_idx(sample_idx.shape[0] - 1, np_rng)
        elif packing_impl == "pack_until_overflow":
            shuffle_idx = np.arange(num_samples)
            np_rng.shuffle(shuffle_idx)
            sample_idx, doc_idx = [], []
            order = np.arange(len(documents))
            np_rng.shuffle(order)
            running, cur = 0, 0
            while len(sample_idx) < num_samples:
                d = documents[order[cur]]
                skip = (not allow_chopped and sizes[d] > seq_length + 1) or \
                    (label_dataset is not None and np.all(label_dataset.get(d)[: seq_length + 1] == -100))
                if not skip:
                    n = int(sizes[d])
                    if running == 0 or running + n > seq_length + 1:
                        sample_idx.append(np.array([len(doc_idx), 0]))
                        running = n
                    else:
                        running += n
                    doc_idx.append(d)
                cur += 1
                if cur == len(documents):
                    cur = 0
                    np_rng.shuffle(order)
            sample_idx.append(np.array([len(doc_idx), 0]))
            doc_idx, sample_idx = np.array(doc_idx), np.array(sample_idx)
        elif packing_impl == "unpacked":
            shuffle_idx = np.arange(num_samples)
            np_rng.shuffle(shuffle_idx)
            sample_idx = np.zeros((num_samples + 1, 2), dtype=np.int64)
            sample_idx[:, 0] = np.arange(num_samples + 1)
            doc_idx, i = [], 0
            while len(doc_idx) <= num_samples:
                d = documents[i]
                skip = (not allow_chopped and sizes[d] > seq_length + 1) or \
                    (label_dataset is not None and np.all(label_dataset.get(d)[:seq_length] == -100))
                if not skip:
                    doc_idx.append(d)
                i = (i + 1) % len(documents)
            doc_idx = np.array(doc_idx)
        else:
            raise ValueError(f"unknown pack_impl {packing_impl}")
        np.save(f_doc, doc_idx, allow_pickle=True)
        np.save(f_sample, sample_idx, allow_pickle=True)
        np.save(f_shuffle, shuffle_idx, allow_pickle=True)
        print_rank_0(f" > elapsed time to build and save index mappings (seconds): {time.time() - t0:4f}")
    _io_barrier()
    doc_idx = np.load(f_doc, allow_pickle=True, mmap_mode="r")
    sample_idx = np.load(f_sample, allow_pickle=True, mmap_mode="r")
    shuffle_idx = np.load(f_shuffle, allow_pickle=True, mmap_mode="r")
    print_rank_0(f"    total number of samples: {sample_idx.shape[0]}")
    print_rank_0(f"    total number of epochs: {num_epochs}")
    return doc_idx, sample_idx, shuffle_idx
