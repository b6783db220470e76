#!/usr/bin/env python
"""Tokenise chat-formatted jsonl with a Hugging Face chat template for SFT / DPO / reward-model / KTO data.

Each line holds a list of ``{"role", "content"}`` messages under ``--jsonl-keys`` (``conversation`` by default).
Outputs ``<prefix>_<key>_document`` (tokens) and ``_label`` (only assistant turns unmasked unless
``--no-mask``); ``--only-last`` unmasks just the final turn (preference data); ``--reward-key`` additionally
writes a per-document reward dataset (KTO).  Mirrors ``tools/datasets/preprocess_data_with_chat_template.py``."""
from __future__ import annotations

import argparse
import json
import sys

import numpy as np

from ...data.indexed_dataset import MMapIndexedDatasetBuilder


def build_chat(chat, tokenizer, generation_role="assistant", apply_mask=True, only_last_turn=False):
    tokens, mask = [], []
    for i, turn in enumerate(chat):
        add_gen = bool(i < len(chat) - 1 and chat[i + 1]["role"] == generation_role)
        ids = tokenizer.apply_chat_template(chat[: i + 1], add_generation_prompt=add_gen, tokenize=True)
        ids = list(ids["input_ids"] if isinstance(ids, dict) else ids)[len(tokens):]
        train_on = (not apply_mask) or (turn["role"] == generation_role and (not only_last_turn or i == len(chat) - 1))
        tokens.extend(ids)
        mask.extend([train_on] * len(ids))
    if tokenizer.eos_token_id is not None:
        tokens.append(tokenizer.eos_token_id)
        mask.append(mask[-1] if mask else True)
    return tokens, mask


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True)
    p.add_argument("--jsonl-keys", nargs="+", default=["conversation"])
    p.add_argument("--no-mask", action="store_true")
    p.add_argument("--generation-role", default="assistant")
    p.add_argument("--only-last", action="store_true")
    p.add_argument("--reward-key", default=None)
    p.add_argument("--tokenizer-path", required=True, help="Hugging Face tokenizer (directory or name) with a chat template")
    p.add_argument("--output-prefix", required=True)
    p.add_argument("--num-docs", type=int, default=None)
    a = p.parse_args(argv)
    from transformers import AutoTokenizer
    tok = AutoTokenizer.from_pretrained(a.tokenizer_path)
    for key in a.jsonl_keys:
        tb = MMapIndexedDatasetBuilder(f"{a.output_prefix}_{key}_document.bin", dtype=np.int32)
        lb = MMapIndexedDatasetBuilder(f"{a.output_prefix}_{key}_document_label.bin", dtype=np.int32)
        rb = MMapIndexedDatasetBuilder(f"{a.output_prefix}_{key}_document_reward.bin", dtype=np.float32) if a.reward_key else None
        n = 0
        for f in a.input.split(","):
            with open(f) as fh:
                for line in fh:
                    if not line.strip():
                        continue
                    doc = json.loads(line)
                    ids, m = build_chat(doc[key], tok, a.generation_role, not a.no_mask, a.only_last)
                    tb.add_item(np.array(ids, dtype=np.int32)); tb.end_document()
                    lb.add_item(np.where(np.array(m), np.array(ids), -100).astype(np.int32)); lb.end_document()
                    if rb is not None:
                        rb.add_item(np.array([doc[a.reward_key]], dtype=np.float32)); rb.end_document()
                    n += 1
                    if a.num_docs and n >= a.num_docs:
                        break
        tb.finalize(f"{a.output_prefix}_{key}_document.idx")
        lb.finalize(f"{a.output_prefix}_{key}_document_label.idx")
        if rb is not None:
            rb.finalize(f"{a.output_prefix}_{key}_document_reward.idx")
    return 0


if __name__ == "__main__":
    sys.exit(main())
