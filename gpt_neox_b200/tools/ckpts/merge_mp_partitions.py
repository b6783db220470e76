#!/usr/bin/env python
"""Merge (or re-split) the tensor-parallel shards of a per-layer checkpoint to another degree, offline
(the generalisation of the reference's ``tools/ckpts/merge20b.py``, which merges the 20B checkpoint from 2 shards to 1).

    python -m gpt_neox_b200.tools.ckpts.merge_mp_partitions --input_dir ckpt/global_step150000 --output_dir merged \\
        --from_mp 2 --to_mp 1
"""
from __future__ import annotations

import argparse
import os
import re

import torch

ROW_WEIGHTS = ("attention.dense.weight", "mlp.linear2.weight", "mlp.dense_4h_to_h.weight")
ROW_BIASES = ("attention.dense.bias", "mlp.linear2.bias", "mlp.dense_4h_to_h.bias")
REPLICATED = ("norm", "layernorm", "inv_freq", "position_embeddings")


def merge_tensors(name, tensors):
    if any(t in name for t in REPLICATED):
        return sum(t.float() for t in tensors).div(len(tensors)).to(tensors[0].dtype)
    if name.endswith(ROW_WEIGHTS):
        return torch.cat(tensors, dim=1)
    if name.endswith(ROW_BIASES):
        return sum(tensors)
    return torch.cat(tensors, dim=0)


def split_tensor(name, tensor, n):
    if any(t in name for t in REPLICATED):
        return [tensor.clone() for _ in range(n)]
    if name.endswith(ROW_WEIGHTS):
        return [c.contiguous() for c in torch.chunk(tensor, n, dim=1)]
    if name.endswith(ROW_BIASES):
        return [tensor / n for _ in range(n)]
    return [c.contiguous() for c in torch.chunk(tensor, n, dim=0)]


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_dir", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--from_mp", type=int, required=True)
    ap.add_argument("--to_mp", type=int, default=1)
    a = ap.parse_args(argv)
    os.makedirs(a.output_dir, exist_ok=True)
    layers = sorted({int(m.group(1)) for f in os.listdir(a.input_dir)
                     if (m := re.match(r"layer_(\d+)-model_\d+-model_states.pt", f))})
    for idx in layers:
        parts = [torch.load(os.path.join(a.input_dir, f"layer_{idx:02d}-model_{r:02d}-model_states.pt"),
                            map_location="cpu", weights_only=False) for r in range(a.from_mp)]
        merged = {k: merge_tensors(k, [p[k] for p in parts]) for k in parts[0]}
        outs = [dict() for _ in range(a.to_mp)]
        for k, v in merged.items():
            for r, piece in enumerate(split_tensor(k, v, a.to_mp)):
                outs[r][k] = piece
        for r, sd in enumerate(outs):
            torch.save(sd, os.path.join(a.output_dir, f"layer_{idx:02d}-model_{r:02d}-model_states.pt"))
    print(f"re-partitioned {len(layers)} layers from mp={a.from_mp} to mp={a.to_mp}")


if __name__ == "__main__":
    main()
