#!/usr/bin/env python
"""Concatenate every ``.bin``/``.idx`` pair found in a directory into one dataset
(``tools/datasets/merge_datasets.py`` of the reference)."""
from __future__ import annotations

import argparse
import os
import sys

from ...data.indexed_dataset import MMapIndexedDataset, MMapIndexedDatasetBuilder


def main(argv=None):
    p = argparse.ArgumentParser()
    p.add_argument("--input", required=True, help="directory holding the datasets to merge")
    p.add_argument("--output-prefix", required=True)
    a = p.parse_args(argv)
    prefixes = sorted({os.path.join(a.input, os.path.splitext(f)[0]) for f in os.listdir(a.input) if f.endswith(".bin")})
    prefixes = [p_ for p_ in prefixes if MMapIndexedDataset.exists(p_)]
    assert prefixes, f"no .bin/.idx pairs in {a.input}"
    builder = None
    for pre in prefixes:
        if builder is None:
            builder = MMapIndexedDatasetBuilder(a.output_prefix + ".bin", dtype=MMapIndexedDataset(pre).dtype)
        builder.merge_file_(pre)
    builder.finalize(a.output_prefix + ".idx")
    print(f"merged {len(prefixes)} datasets into {a.output_prefix}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
