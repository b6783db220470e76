"""Data pipeline: on-disk format, C++ index builders vs their Python twins, packing, blending, samplers, the
preprocessing tool."""
import json
import os
import struct

import numpy as np
import pytest
import torch

from gpt_neox_b200.data import helpers
from gpt_neox_b200.data.blendable_dataset import BlendableDataset
from gpt_neox_b200.data.gpt2_dataset import GPT2Dataset
from gpt_neox_b200.data.indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder, make_dataset
from gpt_neox_b200.data.samplers import DistributedBatchSampler


def _write_corpus(prefix, docs, dtype=np.uint16):
    b = MMapIndexedDatasetBuilder(prefix + ".bin", dtype=dtype)
    for d in docs:
        b.add_item(np.array(d, dtype=dtype))
        b.end_document()
    b.finalize(prefix + ".idx")


def test_mmap_format_round_trip(tmp_path):
    rng = np.random.default_rng(0)
    docs = [rng.integers(0, 1000, size=rng.integers(1, 50)).tolist() for _ in range(30)]
    prefix = str(tmp_path / "corpus")
    _write_corpus(prefix, docs)
    with open(prefix + ".idx", "rb") as fh:
        assert fh.read(9) == b"MMIDIDX\x00\x00"
        assert struct.unpack("<Q", fh.read(8)) == (1,)
        assert struct.unpack("<B", fh.read(1)) == (8,)            # uint16
        assert struct.unpack("<Q", fh.read(8)) == (30,)
        assert struct.unpack("<Q", fh.read(8)) == (31,)
    ds = make_dataset(prefix, "infer")
    assert isinstance(ds, MMapIndexedDataset) and len(ds) == 30
    for i, d in enumerate(docs):
        assert ds[i].tolist() == d
        assert ds.get(i, offset=min(1, len(d) - 1)).tolist() == d[min(1, len(d) - 1):]
    assert [a.tolist() for a in ds[3:6]] == docs[3:6]


def test_cpp_sample_idx_matches_python():
    rng = np.random.default_rng(1)
    sizes = rng.integers(1, 40, size=200).astype(np.int32)
    doc_idx = np.concatenate([rng.permutation(200) for _ in range(3)]).astype(np.int32)
    tokens_per_epoch = int(sizes.sum())
    for seq in (8, 31, 64):
        a = helpers.build_sample_idx(sizes, doc_idx, seq, 3, tokens_per_epoch)
        b = helpers.build_sample_idx_py(sizes, doc_idx, seq, 3, tokens_per_epoch)
        assert np.array_equal(a, b)
        assert a.shape == ((3 * tokens_per_epoch - 1) // seq + 1, 2)


def test_cpp_blending_matches_python_and_weights():
    w = [0.5, 0.3, 0.2]
    a_idx, a_s = helpers.build_blending_indices(w, 1000)
    b_idx, b_s = helpers.build_blending_indices_py(w, 1000)
    assert np.array_equal(a_idx, b_idx) and np.array_equal(a_s, b_s)
    frac = np.bincount(a_idx, minlength=3) / 1000
    assert np.allclose(frac, w, atol=0.01)


@pytest.mark.parametrize("pack_impl", ["packed", "pack_until_overflow", "unpacked"])
def test_gpt2_dataset_packing(tmp_path, pack_impl):
    rng = np.random.default_rng(2)
    docs = [rng.integers(1, 500, size=rng.integers(5, 60)).tolist() for _ in range(64)]
    prefix = str(tmp_path / "c")
    _write_corpus(prefix, docs)
    ds = make_dataset(prefix, "mmap")
    g = GPT2Dataset("train", prefix, np.arange(64, dtype=np.int32), ds, num_samples=50, num_epochs=None,
                    seq_length=32, seed=7, pack_impl=pack_impl)
    assert len(g) >= 49
    x = g[0]["text"]
    assert x.shape == (33,) and x.dtype == np.int64
    if pack_impl == "packed":
        flat = np.concatenate([np.array(docs[d]) for d in g.doc_idx[: 40]])
        assert np.array_equal(g.__getitem__(int(np.where(g.shuffle_idx == 0)[0][0]))["text"], flat[:33])
    # index files are cached next to the data and reused
    n_files = len([f for f in os.listdir(tmp_path) if f.endswith(".npy")])
    GPT2Dataset("train", prefix, np.arange(64, dtype=np.int32), ds, 50, None, 32, 7, pack_impl=pack_impl)
    assert len([f for f in os.listdir(tmp_path) if f.endswith(".npy")]) == n_files == 3


def test_blendable_and_sampler():
    class Const(torch.utils.data.Dataset):
        def __init__(self, v, n):
            self.v, self.n = v, n

        def __len__(self):
            return self.n

        def __getitem__(self, i):
            return self.v

    b = BlendableDataset([Const(0, 700), Const(1, 300)], [0.7, 0.3])
    vals = [b[i] for i in range(len(b))]
    assert abs(sum(vals) / len(vals) - 0.3) < 0.01
    seen = []
    for rank in range(2):
        s = DistributedBatchSampler(torch.utils.data.SequentialSampler(range(16)), batch_size=4, drop_last=True,
                                    rank=rank, world_size=2)
        seen.append(list(s))
    assert seen[0] == [[0, 1], [4, 5], [8, 9], [12, 13]] and seen[1] == [[2, 3], [6, 7], [10, 11], [14, 15]]
    s = DistributedBatchSampler(torch.utils.data.SequentialSampler(range(16)), 4, True, rank=0, world_size=2)
    s.start_iter = 2
    assert list(s) == [[8, 9], [12, 13]]


def test_preprocess_tool_and_mask(tmp_path):
    from gpt_neox_b200.tools.datasets import preprocess_data
    from gpt_neox_b200.tools.datasets.preprocess_data_with_mask import kmp_last_match, mask
    src = tmp_path / "in.jsonl"
    texts = ["hello world", "the quick brown fox", "abc"]
    src.write_text("\n".join(json.dumps({"text": t}) for t in texts))
    out = str(tmp_path / "tok")
    preprocess_data.main(["--input", str(src), "--output-prefix", out, "--tokenizer-type", "CharLevelTokenizer",
                          "--append-eod"])
    ds = make_dataset(out + "_text_document", "mmap")
    assert len(ds) == 3
    assert bytes(ds[0][:-1].astype(np.uint8)).decode() == "hello world" and ds[0][-1] == 0
    assert kmp_last_match([1, 2, 3, 1, 2, 3, 4], [1, 2, 3]) == 6
    assert mask([5, 1, 2, 9, 9], [1, 2]).tolist() == [-100, -100, -100, 9, 9]


def test_tokenizers(tmp_path):
    from types import SimpleNamespace
    from gpt_neox_b200.tokenizer import build_tokenizer
    # a small byte-level BPE vocabulary trained on the spot stands in for a downloaded GPT-2 tokenizer file
    from gpt_neox_b200.tokenizer.train_tokenizer import train_tokenizer
    corpus = tmp_path / "corpus"
    corpus.mkdir()
    with open(corpus / "a.jsonl", "w") as fh:
        for i in range(300):
            fh.write(json.dumps({"text": f"Hello, world! The quick brown fox's {i} jumps\n over  lazy dogs."}) + "\n")
    ref = str(tmp_path / "tok.json")
    train_tokenizer(str(corpus), ref, vocab_size=600)
    args = SimpleNamespace(tokenizer_type="CharLevelTokenizer", make_vocab_size_divisible_by=128, model_parallel_size=2,
                           rank=0, vocab_file=None, merge_file=None)
    t = build_tokenizer(args)
    assert args.padded_vocab_size == 512 and t.detokenize(t.tokenize("abc")) == "abc"
    if os.path.exists(ref):
        args = SimpleNamespace(tokenizer_type="HFTokenizer", make_vocab_size_divisible_by=128, model_parallel_size=1,
                               rank=0, vocab_file=ref, merge_file=None)
        t = build_tokenizer(args)
        ids = t.tokenize("Hello, world!")
        assert t.detokenize(ids) == "Hello, world!" and args.padded_vocab_size % 128 == 0
        # the hand-written byte-level BPE must agree with the tokenizers library on the same vocabulary
        blob = json.load(open(ref))
        vocab, merges = blob["model"]["vocab"], blob["model"]["merges"]
        (tmp_path / "vocab.json").write_text(json.dumps(vocab))
        (tmp_path / "merges.txt").write_text("#version\n" + "\n".join(m if isinstance(m, str) else " ".join(m) for m in merges))
        args = SimpleNamespace(tokenizer_type="GPT2BPETokenizer", make_vocab_size_divisible_by=128, model_parallel_size=1,
                               rank=0, vocab_file=str(tmp_path / "vocab.json"), merge_file=str(tmp_path / "merges.txt"))
        mine = build_tokenizer(args)
        for s in ["Hello, world!", "The quick brown fox's 123 jumps\n over  lazy dogs."]:
            assert mine.tokenize(s) == t.tokenize(s)
            assert mine.detokenize(mine.tokenize(s)) == s


def _pretrain_on_disk(rank, world, cfg):
    from common import make_args
    from gpt_neox_b200.training import pretrain
    args = make_args(**{**cfg, "global_num_gpus": world})
    args.configure_distributed_args()
    pretrain(args)
    assert args.iteration == (cfg.get("train_iters") or args.train_iters) and args.iteration > 0


_ON_DISK_CASES = [
    (2, {"model_parallel_size": 2, "split": "80,10,10"}),                     # only tensor-parallel rank 0 loads data
    (2, {"pipe_parallel_size": 2, "num_layers": 4, "gradient_accumulation_steps": 2, "weight_by_num_documents": True,
         "weighted_sampler_alpha": 0.5, "paths": True}),                      # first and last stage load; 2 / 1 / 1 corpora
    (2, {"train_iters": None, "train_epochs": 1, "split": "60,20,20", "lr_decay_fraction": 0.9}),
]


def test_pretrain_reads_indexed_datasets_from_disk(tmp_path):
    """``pretrain`` end to end on memory-mapped corpora: index files are built once by rank 0 while the other
    data-loading ranks (not the whole world) wait; blended corpora; epochs instead of iterations."""
    from common import run_distributed_many
    jobs = []
    for i, (world, extra) in enumerate(_ON_DISK_CASES):
        d = tmp_path / f"case{i}"
        os.makedirs(d)
        jobs.append((_pretrain_on_disk, world, _on_disk_config(d, extra)))
    run_distributed_many(*jobs, timeout=240)
    for i in range(len(jobs)):
        d = tmp_path / f"case{i}"
        assert os.path.exists(d / "ckpt" / "latest")
        assert any("indexmap" in f for f in os.listdir(d))


def _on_disk_config(tmp_path, extra):
    rng = np.random.default_rng(0)
    for name in ("a", "b"):
        _write_corpus(str(tmp_path / name), [rng.integers(1, 500, size=rng.integers(20, 90)) for _ in range(60)])
    extra = dict(extra)
    cfg = {"save": str(tmp_path / "ckpt"), "train_iters": 6, "lr_decay_iters": 6, "eval_interval": 3, "eval_iters": 2,
           "log_interval": 2, "checkpoint_factor": 3, "num_workers": 0}
    if extra.pop("paths", False):
        cfg.update({"data_path": None, "train_data_paths": [str(tmp_path / "a"), str(tmp_path / "b")],
                    "valid_data_paths": [str(tmp_path / "a")], "test_data_paths": [str(tmp_path / "b")]})
    else:
        cfg["data_path"] = str(tmp_path / "a")
    if extra.get("train_epochs"):
        cfg.pop("lr_decay_iters")
    cfg.update(extra)
    return cfg


def test_pretrain_with_label_pairwise_and_reward_corpora(tmp_path):
    """The side corpora of fine-tuning and preference training through ``pretrain``: per-token labels (SFT masks),
    chosen / rejected pairs (DPO, ``dataset_impl: pairwise``) and per-token rewards (KTO)."""
    from common import run_distributed_many
    jobs = []
    for kind in ("labels", "pairwise", "reward"):
        os.makedirs(tmp_path / kind)
        jobs.append((_pretrain_on_disk, 2, _side_corpora_config(tmp_path / kind, kind)))
    run_distributed_many(*jobs, timeout=240)
    for kind in ("labels", "pairwise", "reward"):
        assert os.path.exists(tmp_path / kind / "ckpt" / "latest")


def _side_corpora_config(tmp_path, kind):
    rng = np.random.default_rng(0)
    docs = [rng.integers(1, 500, size=rng.integers(20, 60)) for _ in range(60)]
    p = lambda n: [str(tmp_path / n)]
    cfg = {"save": str(tmp_path / "ckpt"), "train_iters": 4, "lr_decay_iters": 4, "eval_interval": 2, "eval_iters": 1,
           "log_interval": 2, "checkpoint_factor": 4, "num_workers": 0, "data_path": None, "pack_impl": "unpacked"}
    three = lambda key, n: {f"train_{key}": p(n), f"valid_{key}": p(n), f"test_{key}": p(n)}
    if kind == "pairwise":
        _write_corpus(str(tmp_path / "pos"), docs)
        _write_corpus(str(tmp_path / "neg"), [d[::-1] for d in docs])
        cfg.update({"train_impl": "dpo", "dataset_impl": "pairwise", "dpo_reference_free": True,
                    "train_micro_batch_size_per_gpu": 2})
        for split in ("train", "valid", "test"):
            cfg[f"pos_{split}_data_paths"], cfg[f"neg_{split}_data_paths"] = p("pos"), p("neg")
    else:
        _write_corpus(str(tmp_path / "a"), docs)
        cfg.update({**three("data_paths", "a"), "model_parallel_size": 2})
        if kind == "labels":
            _write_corpus(str(tmp_path / "a_label"), [np.where(np.arange(len(d)) < 3, -100, d) for d in docs],
                          dtype=np.int32)
            cfg.update(three("label_data_paths", "a_label"))
        else:
            _write_corpus(str(tmp_path / "a_reward"),
                          [np.full(len(d), 1.0 if i % 2 else -1.0, dtype=np.float32) for i, d in enumerate(docs)],
                          dtype=np.float32)
            cfg.update({**three("reward_data_paths", "a_reward"), "train_impl": "kto",
                        "train_micro_batch_size_per_gpu": 2})
    return cfg
