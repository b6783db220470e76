#!/usr/bin/env python
"""Look inside checkpoint files, or compare two checkpoints (``tools/ckpts/inspect_checkpoints.py`` of the reference).

    python -m gpt_neox_b200.tools.ckpts.inspect_checkpoints <file-or-dir> [--attributes module/sequential.2.x ...]
                                                             [--stats] [-i]
    python -m gpt_neox_b200.tools.ckpts.inspect_checkpoints -c <dirA>,<dirB> [-d] [--attributes ...]

Every ``.pt`` / ``.ckpt`` file of a directory (natural order: ``layer_2`` before ``layer_10``) is flattened into
``path: description`` lines -- tensors as shape / dtype (``--stats`` adds min / max / mean / norm), scalars and short
containers by value.  ``--attributes`` restricts the listing to sub-trees, nesting written with ``/``.  In compare mode
the files present under both directories are paired by name and every path is marked equal, different (with the largest
absolute difference for tensors of one shape) or present on one side only; ``-d`` prints only what differs.  ``-i`` drops
into a Python shell holding the loaded objects.
"""
from __future__ import annotations

import argparse
import code
import os
import re
from argparse import Namespace
from collections.abc import Mapping

import torch


def natural_key(path):
    """Sort key that orders embedded integers numerically."""
    return [int(t) if t.isdigit() else t.lower() for t in re.split(r"(\d+)", os.path.basename(str(path)))]


def checkpoint_files(path):
    if os.path.isfile(path):
        assert path.endswith((".pt", ".ckpt")), f"{path}: expected a .pt or .ckpt file"
        return [path]
    if not os.path.isdir(path):
        raise ValueError(f"{path}: no such file or directory")
    found = [os.path.join(r, f) for r, _, fs in os.walk(path) for f in fs if f.endswith((".pt", ".ckpt"))]
    return sorted(found, key=lambda f: (os.path.dirname(f), natural_key(f)))


def select(obj, attribute):
    """Follow ``a/b/c`` through mappings, namespaces, sequences (integer parts) and plain attributes."""
    cur = obj
    for part in attribute.split("/"):
        if isinstance(cur, Mapping):
            cur = cur[part] if part in cur else cur[int(part)]
        elif isinstance(cur, (list, tuple)):
            cur = cur[int(part)]
        elif isinstance(cur, Namespace):
            cur = vars(cur)[part]
        else:
            cur = getattr(cur, part)
    return cur


def flatten(obj, prefix="", out=None):
    """``{path: leaf}`` for every tensor / scalar / short container below ``obj``."""
    out = {} if out is None else out
    if isinstance(obj, Mapping) and len(obj):
        for k, v in obj.items():
            flatten(v, f"{prefix}/{k}" if prefix else str(k), out)
    elif isinstance(obj, Namespace):
        flatten(vars(obj), prefix, out)
    elif isinstance(obj, (list, tuple)) and len(obj) and not isinstance(obj[0], (int, float, str, bool, type(None))):
        for i, v in enumerate(obj):
            flatten(v, f"{prefix}/{i}", out)
    else:
        out[prefix] = obj
    return out


def describe_leaf(v, stats=False):
    if torch.is_tensor(v):
        line = f"tensor {tuple(v.shape)} {str(v.dtype).replace('torch.', '')}"
        if stats and v.numel() and (v.is_floating_point() or v.dtype in (torch.int32, torch.int64)):
            f = v.float()
            line += f" min={f.min():.4g} max={f.max():.4g} mean={f.mean():.4g} norm={f.norm():.4g}"
        return line
    s = repr(v)
    return f"{type(v).__name__} {s[:120]}{'...' if len(s) > 120 else ''}"


def describe(obj, attributes=None, stats=False):
    """Lines of one loaded checkpoint object, optionally restricted to ``attributes``."""
    roots = {a: select(obj, a) for a in attributes} if attributes else {"": obj}
    lines = []
    for root, sub in roots.items():
        for path, leaf in flatten(sub, root).items():
            lines.append(f"{path}: {describe_leaf(leaf, stats)}")
    return lines


def _leaf_equal(a, b):
    if torch.is_tensor(a) and torch.is_tensor(b):
        if a.shape != b.shape or a.dtype != b.dtype:
            return False, f"{describe_leaf(a)}  vs  {describe_leaf(b)}"
        if torch.equal(a, b):
            return True, ""
        return False, f"max |a - b| = {(a.double() - b.double()).abs().max().item():.6g}"
    if torch.is_tensor(a) or torch.is_tensor(b):
        return False, f"{describe_leaf(a)}  vs  {describe_leaf(b)}"
    try:
        same = bool(a == b)
    except Exception:
        same = repr(a) == repr(b)
    return same, "" if same else f"{describe_leaf(a)}  vs  {describe_leaf(b)}"


def compare_objects(a, b, attributes=None, only_diffs=False):
    """(lines, number of differences) for two loaded checkpoint objects."""
    fa = {}
    fb = {}
    for root in (attributes or [""]):
        flatten(select(a, root) if root else a, root, fa)
        flatten(select(b, root) if root else b, root, fb)
    lines, diffs = [], 0
    for path in list(fa) + [p for p in fb if p not in fa]:
        if path not in fb:
            lines.append(f"- {path}: only in the first ({describe_leaf(fa[path])})")
            diffs += 1
        elif path not in fa:
            lines.append(f"+ {path}: only in the second ({describe_leaf(fb[path])})")
            diffs += 1
        else:
            same, why = _leaf_equal(fa[path], fb[path])
            if not same:
                lines.append(f"! {path}: {why}")
                diffs += 1
            elif not only_diffs:
                lines.append(f"= {path}: {describe_leaf(fa[path])}")
    return lines, diffs


def _load(path):
    return torch.load(path, map_location="cpu", weights_only=False)


def peek(a):
    for f in checkpoint_files(a.dir):
        print(f"== {f}")
        ckpt = _load(f)
        for line in describe(ckpt, a.attributes, a.stats):
            print("  " + line)
        if a.interactive:
            code.interact(banner="The file's contents are in the variable 'checkpoint'.  Ctrl-D to go on.",
                          local={"checkpoint": ckpt, "torch": torch})


def compare(a):
    dirs = [d.strip() for d in a.dir.split(",")]
    assert len(dirs) == 2, "compare mode takes two comma-separated directories or files"
    names = [{os.path.relpath(f, d) if os.path.isdir(d) else os.path.basename(f): f for f in checkpoint_files(d)}
             for d in dirs]
    shared = sorted(set(names[0]) & set(names[1]), key=natural_key)
    for side, other, d in ((0, 1, dirs[0]), (1, 0, dirs[1])):
        for n in sorted(set(names[side]) - set(names[other]), key=natural_key):
            print(f"only under {d}: {n}")
    total = 0
    for n in shared:
        x, y = _load(names[0][n]), _load(names[1][n])
        lines, diffs = compare_objects(x, y, a.attributes, a.diff)
        total += diffs
        if lines or not a.diff:
            print(f"== {n}: {diffs} difference(s)")
            for line in lines:
                print("  " + line)
        if a.interactive:
            code.interact(banner="The two files are in 'selection_1' and 'selection_2'.  Ctrl-D to go on.",
                          local={"selection_1": x, "selection_2": y, "torch": torch})
    print(f"{len(shared)} file(s) compared, {total} difference(s)")
    return total


def main(argv=None):
    ap = argparse.ArgumentParser(description="Inspect or compare checkpoint files")
    ap.add_argument("dir", help="a .pt / .ckpt file, a directory of them, or with -c two of either separated by a comma")
    ap.add_argument("--attributes", nargs="*", default=None,
                    help="sub-trees to show, nesting written with '/', e.g. module/sequential.2.attention.dense.weight")
    ap.add_argument("--stats", action="store_true", help="also print min / max / mean / norm of tensors")
    ap.add_argument("--interactive", "-i", action="store_true", help="open a Python shell on every file")
    ap.add_argument("--compare", "-c", action="store_true", help="compare two comma-separated checkpoints")
    ap.add_argument("--diff", "-d", action="store_true", help="in compare mode print only what differs")
    a = ap.parse_args(argv)
    if a.compare:
        return compare(a)
    return peek(a)


if __name__ == "__main__":
    main()
