"""Train a byte-level BPE tokenizer (Hugging Face ``tokenizers`` JSON) on a folder of jsonl files.

    python -m gpt_neox_b200.tokenizer.train_tokenizer --json_input_dir data/jsonl --tokenizer_output_path tok.json \
        --vocab_size 52000

Pipeline: NFC normalisation, byte-level pre-tokenisation (so every string is representable), BPE merges learned from
the ``text`` field of every line, byte-level decoder, ``<|endoftext|>`` and ``<|padding|>`` as special tokens.  The
result loads with ``tokenizer_type: HFTokenizer``.  Reference: ``megatron/tokenizer/train_tokenizer.py:49-130``.
"""
import argparse
import glob
import json
import os


def json_iterator(input_dir, text_key="text"):
    for path in sorted(glob.glob(os.path.join(input_dir, "*.jsonl"))):
        with open(path) as fh:
            for line in fh:
                line = line.strip()
                if line:
                    yield json.loads(line)[text_key]


def train_tokenizer(input_dir, save_path, tokenizer_type="BPE", vocab_size=52000, text_key="text"):
    from tokenizers import Tokenizer, decoders, models, normalizers, pre_tokenizers, processors, trainers
    if tokenizer_type != "BPE":
        raise NotImplementedError(f"tokenizer type {tokenizer_type} is not supported (only BPE)")
    tok = Tokenizer(models.BPE())
    tok.normalizer = normalizers.NFC()
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False)
    tok.decoder = decoders.ByteLevel()
    tok.post_processor = processors.ByteLevel(trim_offsets=True)
    trainer = trainers.BpeTrainer(vocab_size=vocab_size, special_tokens=["<|endoftext|>", "<|padding|>"],
                                  initial_alphabet=pre_tokenizers.ByteLevel.alphabet())
    tok.train_from_iterator(json_iterator(input_dir, text_key), trainer)
    os.makedirs(os.path.dirname(os.path.abspath(save_path)), exist_ok=True)
    tok.save(save_path, pretty=True)
    return tok


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--json_input_dir", required=True, help="directory of .jsonl files with a text field")
    ap.add_argument("--tokenizer_output_path", required=True)
    ap.add_argument("--tokenizer_type", default="BPE", choices=["BPE"])
    ap.add_argument("-v", "--vocab_size", type=int, default=52000)
    ap.add_argument("--text_key", default="text")
    a = ap.parse_args(argv)
    train_tokenizer(a.json_input_dir, a.tokenizer_output_path, a.tokenizer_type, a.vocab_size, a.text_key)
    print(f"tokenizer saved at {a.tokenizer_output_path}")


if __name__ == "__main__":
    main()
