#!/usr/bin/env python
"""Render ``configs/neox_arguments.md`` from the configuration schema (one section per key group, one entry per
key with type, default and description).  ``python configs/gen_docs.py``"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from gpt_neox_b200.config.schema import FIELDS, GROUPS  # noqa: E402

TITLES = {"parallelism": "Parallelism", "model": "Model", "optimizer": "Optimizer", "lr_scheduler": "LR scheduler",
          "logging": "Logging", "other": "Miscellaneous", "tokenizer": "Tokenizer", "training": "Training",
          "textgen": "Text generation and MoE", "engine": "Engine (batching, precision, ZeRO)", "runner": "Launcher"}


def render():
    out = ["# Configuration keys", "",
           "Generated from `gpt_neox_b200/config/schema.py`; every key may also be written with `-` instead of `_`.", ""]
    for group, names in GROUPS.items():
        out += [f"## {TITLES.get(group, group)}", ""]
        for n in names:
            f = FIELDS[n]
            out.append(f"- **{n}**: {f.type_str() or 'any'}")
            out.append("")
            out.append(f"    Default = {f.default!r}")
            out.append("")
            if f.doc:
                out.append(f"    {f.doc}")
                out.append("")
    return "\n".join(out) + "\n"


if __name__ == "__main__":
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "neox_arguments.md")
    with open(path, "w") as fh:
        fh.write(render())
    print(f"wrote {path}")
