"""Dataset and data-loader construction (role of ``megatron/data/data_utils.py``).

* only tensor-parallel rank 0 of the first and last pipeline stage builds loaders; the
  ``do_train / do_valid / do_test`` flags are broadcast to everybody else;
* a single ``data_path`` is split by document ranges (``split: "969, 30, 1"``); lists of
  ``train/valid/test_data_paths`` are blended with weights (optionally re-derived from document counts
  with ``weighted_sampler_alpha``);
* ``dataset_impl``: ``gpt2`` (causal LM), ``pairwise`` (chosen/rejected for DPO and reward models),
  ``online`` (REINFORCE samples pulled from a TCP data server);
* ``data_path: synthetic`` yields uniform-random token ids without touching the disk (benchmarks);
* ``shift_and_wrap_data_loaders`` fast-forwards the batch sampler on resume and wraps loaders in
  endless iterators.
"""
from __future__ import annotations

import math
from functools import partial

import numpy as np
import torch
import torch.distributed as dist

from ..parallel import mpu
from ..utils import print_rank_0
from .blendable_dataset import BlendableDataset
from .gpt2_dataset import GPT2Dataset
from .indexed_dataset import make_dataset as make_indexed_dataset
from .samplers import DistributedBatchSampler


class SyntheticDataset(torch.utils.data.Dataset):
    """``seq_length + 1`` uniform-random token ids per sample, a pure function of (seed, index)."""

    def __init__(self, num_samples, seq_length, vocab_size, seed=1234):
        self.n, self.seq_length, self.vocab_size, self.seed = int(num_samples), seq_length, vocab_size, seed

    def __len__(self):
        return self.n

    def __getitem__(self, idx):
        rng = np.random.default_rng((self.seed, int(idx)))
        return {"text": rng.integers(0, self.vocab_size, size=self.seq_length + 1, dtype=np.int64)}


def make_data_loader(dataset, neox_args):
    if dataset is None:
        return None
    world_size, rank = mpu.get_data_parallel_world_size(), mpu.get_data_parallel_rank()
    global_batch_size = neox_args.batch_size * world_size
    sampler = torch.utils.data.SequentialSampler(dataset)
    batch_sampler = DistributedBatchSampler(sampler=sampler, batch_size=global_batch_size, drop_last=True, rank=rank,
                                            world_size=world_size)
    return torch.utils.data.DataLoader(dataset, batch_sampler=batch_sampler, num_workers=neox_args.num_workers,
                                       pin_memory=torch.cuda.is_available())


def get_train_valid_test_split_(splits_string, size):
    sep = "," if "," in splits_string else "/" if "/" in splits_string else None
    splits = [float(s) for s in splits_string.split(sep)] if sep else [float(splits_string)]
    splits = (splits + [0.0, 0.0, 0.0])[:3]
    total = sum(splits)
    assert total > 0.0
    idx = [0]
    for s in splits:
        idx.append(idx[-1] + int(round(s / total * float(size))))
    diff = idx[-1] - size
    idx = [idx[0]] + [i - diff for i in idx[1:]]
    assert len(idx) == 4 and idx[-1] == size
    return idx


def build_the_dataset(data_prefix, pos_data_prefix, neg_data_prefix, name, data_impl, pack_impl, dataset_impl,
                      allow_chopped, num_samples, num_epochs, seq_length, seed, skip_warmup, build_index_mappings=True,
                      label_prefix=None, pos_label_prefix=None, neg_label_prefix=None, precompute_model_name=None,
                      reward_prefix=None):
    mk = lambda p: make_indexed_dataset(p, data_impl, skip_warmup) if p is not None else None
    if dataset_impl == "gpt2":
        indexed = mk(data_prefix)
        n_docs = indexed.sizes.shape[0]
        docs = np.arange(n_docs, dtype=np.int32)
        print_rank_0(f"    {name}:\n     no. of documents:{n_docs}")
        return GPT2Dataset(name, data_prefix, docs, indexed, num_samples, num_epochs, seq_length, seed,
                           pack_impl=pack_impl, allow_chopped=allow_chopped, build_index_mappings=build_index_mappings,
                           label_dataset=mk(label_prefix), reward_dataset=mk(reward_prefix),
                           ref_dataset=mk(data_prefix + "_" + precompute_model_name) if precompute_model_name else None)
    if dataset_impl == "pairwise":
        from .pairwise_dataset import PairwiseDataset
        pos, neg = mk(pos_data_prefix), mk(neg_data_prefix)
        n_docs = pos.sizes.shape[0]
        docs = np.arange(n_docs, dtype=np.int32)
        print_rank_0(f"    {name}:\n     no. of documents:{n_docs}")
        return PairwiseDataset(name, pos_data_prefix, docs, pos, neg, num_samples, seq_length, seed,
                               pack_impl=pack_impl, allow_chopped=allow_chopped,
                               build_index_mappings=build_index_mappings, pos_label_dataset=mk(pos_label_prefix),
                               neg_label_dataset=mk(neg_label_prefix),
                               pos_ref_dataset=mk(pos_data_prefix + "_" + precompute_model_name) if precompute_model_name else None,
                               neg_ref_dataset=mk(neg_data_prefix + "_" + precompute_model_name) if precompute_model_name else None)
    raise NotImplementedError(f"dataset_impl={dataset_impl} not implemented")


def build_train_valid_test_datasets(data_prefix, use_shared_fs, data_impl, pack_impl, allow_chopped, splits_string,
                                    train_valid_test_num_samples, train_valid_test_epochs, seq_length, seed,
                                    skip_warmup):
    indexed = make_indexed_dataset(data_prefix, data_impl, skip_warmup)
    n_docs = indexed.sizes.shape[0]
    splits = get_train_valid_test_split_(splits_string, n_docs)
    print_rank_0(" > dataset split:")
    out = []
    for i, name in enumerate(("train", "valid", "test")):
        print_rank_0(f"    {name}:\n     document indices in [{splits[i]}, {splits[i + 1]}) total of "
                     f"{splits[i + 1] - splits[i]} documents")
        ds = None
        if splits[i + 1] > splits[i]:
            docs = np.arange(splits[i], splits[i + 1], dtype=np.int32)
            ds = GPT2Dataset(name, data_prefix, docs, indexed, train_valid_test_num_samples[i],
                             train_valid_test_epochs[i], seq_length, seed, pack_impl=pack_impl,
                             allow_chopped=allow_chopped, use_shared_fs=use_shared_fs)
        out.append(ds)
    return tuple(out)


def get_normalized_weights_and_num_samples(weights, num_samples):
    s = sum(weights)
    assert s > 0.0
    weights = [w / s for w in weights]
    if num_samples is not None:
        # 0.5% headroom so that blending never runs a dataset dry
        per = [int(math.ceil(num_samples * w * 1.005)) for w in weights]
    else:
        per = [None for _ in weights]
    return weights, per


def weights_by_num_docs(l, alpha=0.3):
    """Multinomial sampling weights from document counts, smoothed by ``alpha`` (as used for
    multilingual corpora): p_i ~ (n_i / N)^alpha, then scaled by (1 - p_i) and renormalised."""
    if len(l) == 1:                 # a single corpus: (1 - p) would be zero
        return [1.0]
    total = sum(l)
    unbiased = [i / total for i in l]
    probs = [p ** alpha for p in unbiased]
    z = sum(probs)
    probs = [p / z for p in probs]
    w = [p * (1 - q) for p, q in zip(probs, unbiased)]
    z = sum(w)
    return [x / z for x in w]


def build_weighted_datasets(neox_args, train_num_samples, valid_num_samples, test_num_samples, train_epochs,
                            valid_epochs, test_epochs, build_index_mappings=True):
    train_ds, valid_ds, test_ds = [], [], []
    a = neox_args
    g = lambda lst, i: lst[i] if lst and i < len(lst) else None      # the three splits may list different numbers of corpora
    n = max(len(x) for x in (a.train_data_paths or a.pos_train_data_paths or [],
                             a.valid_data_paths or a.pos_valid_data_paths or [],
                             a.test_data_paths or a.pos_test_data_paths or []))
    common = dict(data_impl=a.data_impl, pack_impl=a.pack_impl, allow_chopped=a.allow_chopped,
                  seq_length=a.seq_length, seed=a.seed, skip_warmup=not a.mmap_warmup,
                  build_index_mappings=build_index_mappings, dataset_impl=a.dataset_impl,
                  precompute_model_name=a.precompute_model_name)
    for i in range(n):
        if g(a.train_data_paths, i) or g(a.pos_train_data_paths, i):
            train_ds.append(build_the_dataset(
                data_prefix=g(a.train_data_paths, i), name=f"train_{i}", num_samples=g(train_num_samples, i),
                num_epochs=train_epochs, label_prefix=g(a.train_label_data_paths, i),
                reward_prefix=g(a.train_reward_data_paths, i), pos_data_prefix=g(a.pos_train_data_paths, i),
                neg_data_prefix=g(a.neg_train_data_paths, i), pos_label_prefix=g(a.pos_train_label_data_paths, i),
                neg_label_prefix=g(a.neg_train_label_data_paths, i), **common))
        if g(a.valid_data_paths, i) or g(a.pos_valid_data_paths, i):
            valid_ds.append(build_the_dataset(
                data_prefix=g(a.valid_data_paths, i), name=f"valid_{i}", num_samples=g(valid_num_samples, i),
                num_epochs=valid_epochs, label_prefix=g(a.valid_label_data_paths, i),
                reward_prefix=g(a.valid_reward_data_paths, i), pos_data_prefix=g(a.pos_valid_data_paths, i),
                neg_data_prefix=g(a.neg_valid_data_paths, i), pos_label_prefix=g(a.pos_valid_label_data_paths, i),
                neg_label_prefix=g(a.neg_valid_label_data_paths, i), **common))
        if g(a.test_data_paths, i) or g(a.pos_test_data_paths, i):
            test_ds.append(build_the_dataset(
                data_prefix=g(a.test_data_paths, i), name=f"test_{i}", num_samples=g(test_num_samples, i),
                num_epochs=test_epochs, label_prefix=g(a.test_label_data_paths, i),
                reward_prefix=g(a.test_reward_data_paths, i), pos_data_prefix=g(a.pos_test_data_paths, i),
                neg_data_prefix=g(a.neg_test_data_paths, i), pos_label_prefix=g(a.pos_test_label_data_paths, i),
                neg_label_prefix=g(a.neg_test_label_data_paths, i), **common))
    return train_ds, valid_ds, test_ds


def validate_train_epochs(neox_args):
    if neox_args.train_epochs is None:
        return
    if neox_args.train_epochs and neox_args.train_iters:
        raise ValueError("Cannot specify both train epochs and train iters simultaneously")
    if neox_args.train_data_weights and not all(w == 1.0 for w in neox_args.train_data_weights):
        raise ValueError("train_epochs currently does not support weighted datasets")


def _synthetic(neox_args):
    return neox_args.data_path == "synthetic" or (neox_args.data_path is None and not neox_args.train_data_paths
                                                  and not neox_args.pos_train_data_paths
                                                  and neox_args.dataset_impl != "online")


def build_train_valid_test_data_loaders(neox_args):
    validate_train_epochs(neox_args)
    train_dl = valid_dl = test_dl = None
    print_rank_0("> building train, validation, and test datasets ...")
    if neox_args.is_pipe_parallel:
        pipe_load = mpu.is_pipeline_first_stage() or mpu.is_pipeline_last_stage()
    else:
        pipe_load = True
    a = neox_args
    flags = [0, 0, 0]
    if pipe_load and mpu.get_model_parallel_rank() == 0:
        train_iters = a.train_iters or 0
        eval_every = a.eval_interval or max(train_iters, 1)
        eval_iters_total = (train_iters // eval_every + 1) * a.eval_iters
        nsamp = [train_iters * a.train_batch_size, eval_iters_total * a.train_batch_size, a.eval_iters * a.train_batch_size]
        epochs = [a.train_epochs, None, None]
        if a.train_epochs:
            nsamp = [None, None, None]
            epochs = [a.train_epochs, 1, 1]
        if a.dataset_impl == "online":
            from .online_dataset import OnlineDataset
            mk = lambda split, n: OnlineDataset(leave_one_out=a.reinforce_leave_one_out, data_split=split,
                                                num_samples=n, seq_length=a.seq_length,
                                                dataserver_ips=a.online_dataserver_ips,
                                                dataserver_ports=a.online_dataserver_ports)
            train_ds, valid_ds, test_ds = mk("train", nsamp[0]), mk("valid", nsamp[1]), mk("test", nsamp[2])
        elif _synthetic(a):
            mk = lambda n, s: SyntheticDataset(max(n or 0, a.train_batch_size), a.seq_length, a.padded_vocab_size,
                                               seed=a.seed + s)
            train_ds, valid_ds, test_ds = mk(nsamp[0], 0), mk(nsamp[1], 1), mk(nsamp[2], 2)
        elif a.train_data_paths or a.pos_train_data_paths:
            tw, tn = get_normalized_weights_and_num_samples(a.train_data_weights, nsamp[0])
            vw, vn = get_normalized_weights_and_num_samples(a.valid_data_weights, nsamp[1])
            sw, sn = get_normalized_weights_and_num_samples(a.test_data_weights, nsamp[2])
            tds, vds, sds = build_weighted_datasets(a, tn, vn, sn, epochs[0], epochs[1], epochs[2],
                                                    build_index_mappings=not a.weight_by_num_documents)
            if a.weight_by_num_documents:
                fn = partial(weights_by_num_docs, alpha=a.weighted_sampler_alpha)
                count = lambda dss: [d.indexed_dataset.sizes.shape[0] for d in dss]
                tw, vw, sw = fn(count(tds)), fn(count(vds)), fn(count(sds))
                tw, tn = get_normalized_weights_and_num_samples(tw, nsamp[0])
                vw, vn = get_normalized_weights_and_num_samples(vw, nsamp[1])
                sw, sn = get_normalized_weights_and_num_samples(sw, nsamp[2])
                tds, vds, sds = build_weighted_datasets(a, tn, vn, sn, epochs[0], epochs[1], epochs[2])
            blend = lambda dss, w: BlendableDataset(dss, w) if dss else None
            train_ds, valid_ds, test_ds = blend(tds, tw), blend(vds, vw), blend(sds, sw)
        else:
            train_ds, valid_ds, test_ds = build_train_valid_test_datasets(
                data_prefix=a.data_path, use_shared_fs=a.use_shared_fs, data_impl=a.data_impl, pack_impl=a.pack_impl,
                allow_chopped=a.allow_chopped, splits_string=a.split, train_valid_test_num_samples=nsamp,
                train_valid_test_epochs=epochs, seq_length=a.seq_length, seed=a.seed, skip_warmup=not a.mmap_warmup)
        train_dl, valid_dl, test_dl = (make_data_loader(d, a) for d in (train_ds, valid_ds, test_ds))
        if a.train_epochs:
            flags = [int(train_dl is not None), int(valid_dl is not None), int(test_dl is not None)]
        else:
            flags = [int(train_dl is not None and train_iters > 0), int(valid_dl is not None and a.eval_iters > 0),
                     int(test_dl is not None and a.eval_iters > 0)]
    if dist.is_available() and dist.is_initialized():
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        t = torch.tensor(flags, dtype=torch.long, device=dev)
        if a.is_pipe_parallel:
            dist.broadcast(t, src=0)
        else:
            dist.broadcast(t, mpu.get_model_parallel_src_rank(), group=mpu.get_model_parallel_group())
        flags = t.tolist()
    a.do_train, a.do_valid, a.do_test = bool(flags[0]), bool(flags[1]), bool(flags[2])
    return train_dl, valid_dl, test_dl


def shift_and_wrap_data_loaders(neox_args, train_dl, valid_dl, test_dl, loop=True):
    for name, dl in (("training", train_dl), ("validation", valid_dl), ("test", test_dl)):
        if dl is not None and len(dl) == 0:
            raise ValueError(f"the {name} split holds fewer samples than one batch per data-parallel rank "
                             "(check `split` / the data paths / train_micro_batch_size_per_gpu)")
    if train_dl is not None:
        train_dl.batch_sampler.start_iter = (neox_args.iteration * neox_args.gradient_accumulation_steps) % len(train_dl)
        print_rank_0(f"setting training data start iteration to {train_dl.batch_sampler.start_iter}")
    if valid_dl is not None and neox_args.eval_interval:
        start = ((neox_args.iteration * neox_args.gradient_accumulation_steps) // neox_args.eval_interval) \
            * neox_args.eval_iters
        valid_dl.batch_sampler.start_iter = start % len(valid_dl)
        print_rank_0(f"setting validation data start iteration to {valid_dl.batch_sampler.start_iter}")

    def endless(dl):
        while True:
            for x in dl:
                yield x

    wrap = (lambda dl: endless(dl)) if loop else iter
    return tuple(wrap(dl) if dl is not None else None for dl in (train_dl, valid_dl, test_dl))
