#!/usr/bin/env python
"""Download (when a network is available) and tokenise a named corpus into ``.bin``/``.idx`` files
(``prepare_data.py:29-77`` of the reference)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

TOKENIZER_CHOICES = ["HFGPT2Tokenizer", "HFTokenizer", "GPT2BPETokenizer", "CharLevelTokenizer", "TiktokenTokenizer",
                     "SPMTokenizer"]


def get_args(input_args=None):
    from gpt_neox_b200.tools.datasets.corpora import DATA_DOWNLOADERS
    p = argparse.ArgumentParser(description="Download & preprocess neox datasets")
    p.add_argument("dataset", nargs="?", default="enwik8", choices=list(DATA_DOWNLOADERS) + ["all"],
                   help="name of dataset to download.")
    p.add_argument("-t", "--tokenizer", default="GPT2BPETokenizer", choices=TOKENIZER_CHOICES)
    p.add_argument("-d", "--data-dir", default=None, help="Directory to which to download datasets / tokenizer "
                                                           "files - defaults to ./data")
    p.add_argument("-v", "--vocab-file", default=None)
    p.add_argument("-m", "--merge-file", default=None)
    p.add_argument("-f", "--force-redownload", dest="force_redownload", default=False, action="store_true")
    return p.parse_args(input_args)


def main(input_args=None):
    from gpt_neox_b200.tools.datasets.corpora import prepare_dataset
    args = get_args(input_args)
    prepare_dataset(dataset_name=args.dataset, tokenizer_type=args.tokenizer, data_dir=args.data_dir,
                    vocab_file=args.vocab_file, merge_file=args.merge_file, force_redownload=args.force_redownload)


if __name__ == "__main__":
    main()
