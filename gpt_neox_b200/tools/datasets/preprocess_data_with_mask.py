#!/usr/bin/env python
"""Like ``preprocess_data`` but also writes a ``_label`` dataset in which everything up to (and including) the last
occurrence of a pivot string is masked with ``-100`` -- e.g. mask the prompt, train on the answer.
``--mask-before-token`` accepts comma-separated token ids (the pivot); the pivot is located with the
Knuth-Morris-Pratt matcher below (``tools/datasets/preprocess_data_with_mask.py`` of the reference)."""
from __future__ import annotations

import sys

import numpy as np

from ...data.indexed_dataset import make_builder
from ...tokenizer import build_tokenizer
from . import preprocess_data as P


def kmp_last_match(seq, pat):
    """Index one past the LAST occurrence of ``pat`` in ``seq`` (-1 if absent)."""
    if not pat:
        return -1
    fail, k = [0] * len(pat), 0
    for i in range(1, len(pat)):
        while k and pat[i] != pat[k]:
            k = fail[k - 1]
        if pat[i] == pat[k]:
            k += 1
        fail[i] = k
    last, k = -1, 0
    for i, s in enumerate(seq):
        while k and s != pat[k]:
            k = fail[k - 1]
        if s == pat[k]:
            k += 1
        if k == len(pat):
            last = i + 1
            k = fail[k - 1]
    return last


def mask(tokens, pivot):
    labels = np.array(tokens, dtype=np.int64)
    end = kmp_last_match(list(tokens), pivot)
    if end > 0:
        labels[:end] = -100
    return labels


def main(argv=None):
    argv = list(argv if argv is not None else sys.argv[1:])
    pivot = []
    if "--mask-before-token" in argv:
        i = argv.index("--mask-before-token")
        pivot = [int(t) for t in argv[i + 1].split(",")]
        del argv[i:i + 2]
    args = P.get_args(argv)
    tok = build_tokenizer(args)
    key = args.jsonl_keys[0]
    text_b = make_builder(f"{args.output_prefix}_{key}_document.bin", impl="mmap", vocab_size=tok.vocab_size)
    label_b = make_builder(f"{args.output_prefix}_{key}_document_label.bin", impl="mmap", vocab_size=None)
    label_b._dtype = np.int64
    for doc in P.yield_from_files(args.input.split(","), args.jsonl_keys):
        ids = tok.tokenize(doc[key])
        if args.append_eod:
            ids = list(ids) + [tok.eod]
        if not ids:
            continue
        text_b.add_item(np.array(ids, dtype=text_b.dtype))
        text_b.end_document()
        label_b.add_item(mask(ids, pivot))
        label_b.end_document()
    text_b.finalize(f"{args.output_prefix}_{key}_document.idx")
    label_b.finalize(f"{args.output_prefix}_{key}_document_label.idx")
    return 0


if __name__ == "__main__":
    sys.exit(main())
