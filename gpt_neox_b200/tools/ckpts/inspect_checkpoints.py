#!/usr/bin/env python
"""Print the contents of checkpoint files: keys, tensor shapes / dtypes / norms, scalar values
(``tools/ckpts/inspect_checkpoints.py`` of the reference).  ``python -m ...inspect_checkpoints <file-or-dir> [--attributes]``"""
from __future__ import annotations

import argparse
import os

import torch


def describe(obj, prefix="", out=None, attributes=False):
    out = out if out is not None else []
    if torch.is_tensor(obj):
        line = f"{prefix}: tensor {tuple(obj.shape)} {obj.dtype}"
        if attributes and obj.numel() and obj.is_floating_point():
            f = obj.float()
            line += f" min={f.min():.4g} max={f.max():.4g} mean={f.mean():.4g} norm={f.norm():.4g}"
        out.append(line)
    elif isinstance(obj, dict):
        for k, v in obj.items():
            describe(v, f"{prefix}.{k}" if prefix else str(k), out, attributes)
    elif isinstance(obj, (list, tuple)) and len(obj) and not isinstance(obj[0], (int, float, str)):
        for i, v in enumerate(obj):
            describe(v, f"{prefix}[{i}]", out, attributes)
    else:
        s = repr(obj)
        out.append(f"{prefix}: {s[:120]}{'...' if len(s) > 120 else ''}")
    return out


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("path")
    ap.add_argument("--attributes", action="store_true", help="also print min / max / mean / norm of tensors")
    a = ap.parse_args(argv)
    files = [a.path] if os.path.isfile(a.path) else sorted(
        os.path.join(r, f) for r, _, fs in os.walk(a.path) for f in fs if f.endswith(".pt"))
    for f in files:
        print(f"== {f}")
        for line in describe(torch.load(f, map_location="cpu", weights_only=False), attributes=a.attributes):
            print("  " + line)


if __name__ == "__main__":
    main()
