"""Count the tokens of one or more indexed (``.bin`` / ``.idx``) datasets.

    python -m gpt_neox_b200.tools.datasets.dataset_token_count data/pile_text_document data/other_text_document

Prints the document count and total token count per dataset prefix (reference:
``tools/datasets/dataset_token_count.py``, which sums the ``sizes`` array of the memory-mapped index).
"""
import argparse

import numpy as np

from ...data.indexed_dataset import make_dataset


def count(prefix, impl="mmap"):
    ds = make_dataset(prefix, impl)
    sizes = np.asarray(ds.sizes, dtype=np.int64)
    return len(sizes), int(sizes.sum())


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("prefixes", nargs="+", help="dataset paths without the .bin / .idx extension")
    ap.add_argument("--impl", default="mmap", choices=["mmap", "lazy", "cached", "infer"])
    a = ap.parse_args(argv)
    total = 0
    for p in a.prefixes:
        docs, toks = count(p, a.impl)
        total += toks
        print(f"{p}: {docs} documents, {toks} tokens")
    if len(a.prefixes) > 1:
        print(f"total: {total} tokens")


if __name__ == "__main__":
    main()
