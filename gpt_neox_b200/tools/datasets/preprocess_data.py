#!/usr/bin/env python
"""Tokenise ``.jsonl`` (optionally ``.jsonl.zst`` / ``.gz``) corpora into the memory-mapped ``.bin`` / ``.idx`` format.

    python -m gpt_neox_b200.tools.datasets.preprocess_data --input data.jsonl --output-prefix data/mycorpus \\
        --tokenizer-type HFTokenizer --vocab-file tokenizer.json --append-eod --workers 8

One document per JSON line (key ``text`` by default, ``--jsonl-keys`` for others); a worker pool tokenises, the
parent appends each document to ``<prefix>_<key>_document.bin`` and finally writes the index.
Same flags as ``tools/datasets/preprocess_data.py`` of the reference.
"""
from __future__ import annotations

import argparse
import gzip
import io
import json
import multiprocessing
import sys
import time

import numpy as np

from ...data.indexed_dataset import make_builder
from ...tokenizer import build_tokenizer


def iter_lines(path):
    if path.endswith(".zst"):
        import zstandard
        with open(path, "rb") as fh:
            reader = io.TextIOWrapper(zstandard.ZstdDecompressor().stream_reader(fh), encoding="utf-8")
            yield from reader
    elif path.endswith(".gz"):
        with gzip.open(path, "rt", encoding="utf-8") as fh:
            yield from fh
    else:
        with open(path, "r", encoding="utf-8") as fh:
            yield from fh


def yield_from_files(paths, keys):
    for path in paths:
        for line in iter_lines(path):
            line = line.strip()
            if not line:
                continue
            if path.endswith((".txt",)):
                yield {keys[0]: line}
            else:
                yield json.loads(line)


class Encoder:
    tokenizer = None

    def __init__(self, args):
        self.args = args

    def initializer(self):
        Encoder.tokenizer = build_tokenizer(self.args)

    def encode(self, doc):
        ids = {}
        n = 0
        for key in self.args.jsonl_keys:
            text = doc[key] if isinstance(doc, dict) else doc
            if self.args.ftfy:
                import ftfy
                text = ftfy.fix_text(text)
            tok = Encoder.tokenizer.tokenize(text)
            if self.args.append_eod:
                tok = list(tok) + [Encoder.tokenizer.eod]
            ids[key] = [tok] if len(tok) > 0 else []
            n += len(text)
        return ids, n


def get_args(argv=None):
    p = argparse.ArgumentParser()
    g = p.add_argument_group("input data")
    g.add_argument("--input", type=str, required=True, help="comma-separated list of jsonl / jsonl.zst / txt files")
    g.add_argument("--jsonl-keys", nargs="+", default=["text"])
    g.add_argument("--num-docs", default=None, type=int)
    g = p.add_argument_group("tokenizer")
    g.add_argument("--tokenizer-type", type=str, required=True,
                   choices=["HFGPT2Tokenizer", "HFTokenizer", "GPT2BPETokenizer", "CharLevelTokenizer", "TiktokenTokenizer",
                            "SPMTokenizer"])
    g.add_argument("--vocab-file", type=str, default=None)
    g.add_argument("--merge-file", type=str, default=None)
    g.add_argument("--append-eod", action="store_true")
    g.add_argument("--ftfy", action="store_true")
    g = p.add_argument_group("output data")
    g.add_argument("--output-prefix", type=str, required=True)
    g.add_argument("--dataset-impl", type=str, default="mmap", choices=["lazy", "cached", "mmap"])
    g = p.add_argument_group("runtime")
    g.add_argument("--workers", type=int, default=1)
    g.add_argument("--log-interval", type=int, default=100)
    a = p.parse_args(argv)
    a.keep_empty = False
    a.rank = 0
    a.make_vocab_size_divisible_by = 128
    a.model_parallel_size = 1
    return a


def main(argv=None):
    args = get_args(argv)
    encoder = Encoder(args)
    tokenizer = build_tokenizer(args)
    docs = yield_from_files(args.input.split(","), args.jsonl_keys)
    if args.workers > 1:
        pool = multiprocessing.Pool(args.workers, initializer=encoder.initializer)
        encoded = pool.imap(encoder.encode, docs, chunksize=25)
    else:
        encoder.initializer()
        encoded = (encoder.encode(d) for d in docs)
    builders, bins, idxs = {}, {}, {}
    for key in args.jsonl_keys:
        bins[key] = f"{args.output_prefix}_{key}_document.bin"
        idxs[key] = f"{args.output_prefix}_{key}_document.idx"
        builders[key] = make_builder(bins[key], impl=args.dataset_impl, vocab_size=tokenizer.vocab_size)
    t0, total = time.time(), 0
    for i, (doc, nbytes) in enumerate(encoded, start=1):
        total += nbytes
        for key, sentences in doc.items():
            for s in sentences:
                builders[key].add_item(np.array(s, dtype=builders[key].dtype))
            builders[key].end_document()
        if i % args.log_interval == 0:
            dt = time.time() - t0
            print(f"Processed {i} documents ({i / dt:.2f} docs/s, {total / dt / 1024 / 1024:.2f} MB/s).", flush=True)
        if args.num_docs and i >= args.num_docs:
            break
    for key in args.jsonl_keys:
        builders[key].finalize(idxs[key])
    return 0


if __name__ == "__main__":
    sys.exit(main())
