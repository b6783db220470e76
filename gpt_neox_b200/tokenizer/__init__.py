"""Tokenizers selectable by ``tokenizer_type`` (reference ``megatron/tokenizer/tokenizer.py:30-404``):
GPT2BPETokenizer (vocab.json + merges.txt, byte-level BPE implemented here), HFTokenizer (a
``tokenizers`` JSON file), HFGPT2Tokenizer (transformers), SPMTokenizer (sentencepiece),
CharLevelTokenizer (raw bytes) and TiktokenTokenizer.

``build_tokenizer(args)`` also sets ``args.padded_vocab_size``: the vocabulary rounded up to a
multiple of ``make_vocab_size_divisible_by * model_parallel_size`` so it shards evenly.
"""
from __future__ import annotations

import json
from abc import ABC, abstractmethod
from functools import lru_cache
from typing import List, Union

import numpy as np


def _vocab_size_with_padding(orig_vocab_size, args):
    multiple = args.make_vocab_size_divisible_by * args.model_parallel_size
    after = orig_vocab_size
    while after % multiple != 0:
        after += 1
    if getattr(args, "rank", 0) in (0, None):
        print(f" > padded vocab (size: {orig_vocab_size}) with {after - orig_vocab_size} dummy tokens "
              f"(new size: {after})", flush=True)
    return after


def build_tokenizer(args):
    if getattr(args, "rank", 0) in (0, None):
        print(f"> building {args.tokenizer_type} tokenizer ...", flush=True)
    t = args.tokenizer_type.lower()
    if t == "gpt2bpetokenizer":
        assert args.vocab_file is not None and args.merge_file is not None
        tok = GPT2BPETokenizer(args.vocab_file, args.merge_file)
    elif t == "spmtokenizer":
        assert args.vocab_file is not None
        tok = SentencePieceTokenizer(args.vocab_file)
    elif t == "hftokenizer":
        assert args.vocab_file is not None
        tok = HFTokenizer(args.vocab_file)
    elif t == "hfgpt2tokenizer":
        if args.vocab_file is None:
            print("WARNING: No vocab file found, loading Huggingface's pretrained GPT2Tokenizer")
        tok = HFGPT2Tokenizer(args.vocab_file)
    elif t == "charleveltokenizer":
        tok = CharLevelTokenizer(vocab_size=512)
    elif t == "tiktokentokenizer":
        assert args.vocab_file is not None
        tok = TiktokenTokenizer(args.vocab_file)
    else:
        raise NotImplementedError(f"{args.tokenizer_type} tokenizer is not implemented.")
    args.padded_vocab_size = _vocab_size_with_padding(tok.vocab_size, args)
    return tok


class AbstractTokenizer(ABC):
    def __init__(self, name):
        self.name = name

    @property
    @abstractmethod
    def vocab_size(self):
        ...

    @property
    @abstractmethod
    def vocab(self):
        ...

    @property
    @abstractmethod
    def inv_vocab(self):
        ...

    @abstractmethod
    def tokenize(self, text):
        ...

    def detokenize(self, token_ids):
        raise NotImplementedError(f"detokenizer is not implemented for {self.name} tokenizer")

    def tokenize_batch(self, texts):
        return [self.tokenize(t) for t in texts]

    @property
    def eod(self):
        raise NotImplementedError

    @property
    def cls(self):
        raise NotImplementedError

    @property
    def sep(self):
        raise NotImplementedError

    @property
    def pad(self):
        raise NotImplementedError

    @property
    def mask(self):
        raise NotImplementedError


@lru_cache()
def bytes_to_unicode():
    """Reversible byte -> printable unicode map used by byte-level BPE."""
    bs = list(range(ord("!"), ord("~") + 1)) + list(range(ord("¡"), ord("¬") + 1)) + list(range(ord("®"), ord("ÿ") + 1))
    cs, n = bs[:], 0
    for b in range(256):
        if b not in bs:
            bs.append(b)
            cs.append(256 + n)
            n += 1
    return dict(zip(bs, [chr(c) for c in cs]))


class GPT2BPETokenizer(AbstractTokenizer):
    """Byte-level BPE from ``vocab.json`` and ``merges.txt`` (GPT-2 pre-tokenisation pattern)."""

    def __init__(self, vocab_file, merge_file):
        super().__init__("GPT2 BPE")
        import regex as re
        with open(vocab_file) as fh:
            self.encoder = json.load(fh)
        self.decoder = {v: k for k, v in self.encoder.items()}
        with open(merge_file, encoding="utf-8") as fh:
            lines = fh.read().split("\n")
        merges = [tuple(l.split()) for l in lines[1:] if l and len(l.split()) == 2]
        self.bpe_ranks = dict(zip(merges, range(len(merges))))
        self.byte_encoder = bytes_to_unicode()
        self.byte_decoder = {v: k for k, v in self.byte_encoder.items()}
        self.pat = re.compile(r"""'s|'t|'re|'ve|'m|'ll|'d| ?\p{L}+| ?\p{N}+| ?[^\s\p{L}\p{N}]+|\s+(?!\S)|\s+""")
        self.cache = {}
        self.eod_id = self.encoder["<|endoftext|>"]

    def _bpe(self, token):
        if token in self.cache:
            return self.cache[token]
        word = tuple(token)
        while len(word) > 1:
            pairs = {(word[i], word[i + 1]) for i in range(len(word) - 1)}
            best = min(pairs, key=lambda p: self.bpe_ranks.get(p, float("inf")))
            if best not in self.bpe_ranks:
                break
            a, b = best
            out, i = [], 0
            while i < len(word):
                if i < len(word) - 1 and word[i] == a and word[i + 1] == b:
                    out.append(a + b)
                    i += 2
                else:
                    out.append(word[i])
                    i += 1
            word = tuple(out)
        res = " ".join(word)
        self.cache[token] = res
        return res

    @property
    def vocab_size(self):
        return len(self.encoder)

    @property
    def vocab(self):
        return self.encoder

    @property
    def inv_vocab(self):
        return self.decoder

    def tokenize(self, text):
        ids = []
        for tok in self.pat.findall(text):
            tok = "".join(self.byte_encoder[b] for b in tok.encode("utf-8"))
            ids.extend(self.encoder[t] for t in self._bpe(tok).split(" "))
        return ids

    def detokenize(self, token_ids):
        text = "".join(self.decoder[int(t)] for t in token_ids)
        return bytearray([self.byte_decoder[c] for c in text]).decode("utf-8", errors="replace")

    @property
    def eod(self):
        return self.eod_id


class SentencePieceTokenizer(AbstractTokenizer):
    def __init__(self, vocab_file):
        super().__init__("SPM")
        import sentencepiece as spm
        self.tokenizer = spm.SentencePieceProcessor(model_file=vocab_file)
        self.eod_id = self.tokenizer.piece_to_id("<|endoftext|>")

    @property
    def vocab_size(self):
        return self.tokenizer.get_piece_size()

    @property
    def vocab(self):
        return {self.tokenizer.id_to_piece(i): i for i in range(self.tokenizer.get_piece_size())}

    @property
    def inv_vocab(self):
        return {i: self.tokenizer.id_to_piece(i) for i in range(self.tokenizer.get_piece_size())}

    def tokenize(self, text):
        return self.tokenizer.encode(text)

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class HFTokenizer(AbstractTokenizer):
    def __init__(self, vocab_file):
        super().__init__("HFTokenizer")
        from tokenizers import Tokenizer
        self.tokenizer = Tokenizer.from_file(vocab_file)
        self.eod_id = self.tokenizer.token_to_id("<|endoftext|>")
        self.pad_id = self.tokenizer.token_to_id("<|padding|>")

    @property
    def vocab_size(self):
        return self.tokenizer.get_vocab_size()

    @property
    def vocab(self):
        return self.tokenizer.get_vocab()

    @property
    def inv_vocab(self):
        return {v: k for k, v in self.tokenizer.get_vocab().items()}

    def tokenize(self, text):
        return self.tokenizer.encode(text).ids

    def tokenize_batch(self, texts):
        return [e.ids for e in self.tokenizer.encode_batch(texts)]

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class HFGPT2Tokenizer(AbstractTokenizer):
    def __init__(self, vocab_file=None, fast=True):
        super().__init__("HFGPT2Tokenizer")
        from transformers import GPT2Tokenizer, GPT2TokenizerFast
        cls = GPT2TokenizerFast if fast else GPT2Tokenizer
        self.tokenizer = cls.from_pretrained(vocab_file or "gpt2")
        self.tokenizer.add_special_tokens({"pad_token": "<|padding|>"})
        self.eod_id = self.tokenizer.eos_token_id
        self.pad_id = self.tokenizer.pad_token_id

    @property
    def vocab_size(self):
        return len(self.tokenizer)

    @property
    def vocab(self):
        return self.tokenizer.get_vocab()

    @property
    def inv_vocab(self):
        return self.tokenizer._tokenizer.decoder

    def tokenize(self, text):
        return self.tokenizer.encode(text)

    def detokenize(self, token_ids):
        return self.tokenizer.decode(list(map(int, token_ids)))

    @property
    def eod(self):
        return self.eod_id


class CharLevelTokenizer(AbstractTokenizer):
    """One token per byte value (clamped into the vocabulary)."""

    def __init__(self, vocab_size):
        super().__init__("CharLevelTokenizer")
        self._vocab_size = vocab_size
        self.eod_id = 0
        self.pad_id = 1

    def clamp(self, n):
        return max(32, min(n, self.vocab_size))

    @property
    def vocab_size(self):
        return self._vocab_size

    @property
    def vocab(self):
        raise NotImplementedError

    @property
    def inv_vocab(self):
        raise NotImplementedError

    def decode_token(self, token):
        return str(chr(self.clamp(int(token))))

    def tokenize(self, text):
        return list(np.frombuffer(text.encode("utf-8", errors="ignore") if isinstance(text, str) else text,
                                  dtype=np.uint8).astype(np.int64))

    def detokenize(self, token_ids):
        return "".join(self.decode_token(t) for t in token_ids)

    @property
    def eod(self):
        return self.eod_id


class TiktokenTokenizer(AbstractTokenizer):
    def __init__(self, vocab_file):
        super().__init__("TiktokenTokenizer")
        import tiktoken
        self.tokenizer = tiktoken.get_encoding(vocab_file)
        self.eod_id = self.tokenizer.eot_token
        self.pad_id = None

    @property
    def vocab_size(self):
        return self.tokenizer.n_vocab

    @property
    def vocab(self):
        raise NotImplementedError("TiktokenTokenizer does not implement vocabulary access.")

    @property
    def inv_vocab(self):
        raise NotImplementedError("TiktokenTokenizer does not implement vocabulary access.")

    def tokenize(self, text):
        return self.tokenizer.encode(text)

    def tokenize_batch(self, texts):
        return self.tokenizer.encode_batch(texts, allowed_special="all")

    def detokenize(self, token_ids):
        return self.tokenizer.decode(tokens=list(map(int, token_ids)), errors="strict")

    @property
    def eod(self):
        return self.eod_id

    @property
    def pad(self):
        raise NotImplementedError
