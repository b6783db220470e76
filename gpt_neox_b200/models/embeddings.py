"""Input embeddings (reference ``megatron/model/word_embeddings.py:24-251``): vocabulary-parallel token
embedding, optional learned / sinusoidal positions (OPT offset supported), token types, dropout, muP
multiplier, and the scatter into the sequence-parallel region along dim 1 (``[b, s, h]``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..parallel import mappings as M
from ..parallel import mpu
from ..parallel.layers import VocabParallelEmbedding
from .positional import SinusoidalPositionalEmbedding


class Embedding(nn.Module):
    def __init__(self, neox_args, hidden_size, vocab_size, max_sequence_length, embedding_dropout_prob, init_method,
                 num_tokentypes=0, use_pos_emb=True):
        super().__init__()
        self.hidden_size, self.init_method, self.num_tokentypes = hidden_size, init_method, num_tokentypes
        self.sequence_parallel = neox_args.sequence_parallel and mpu.get_model_parallel_world_size() > 1
        self.use_mup = neox_args.use_mup
        self.mup_embedding_mult = neox_args.mup_embedding_mult
        self.mup_rp_embedding_mult = neox_args.mup_rp_embedding_mult
        self.word_embeddings = VocabParallelEmbedding(neox_args, vocab_size, hidden_size, init_method=init_method)
        dev = self.word_embeddings.weight.device
        self.use_pos_emb = use_pos_emb
        self.embedding_type = neox_args.pos_emb if use_pos_emb else None
        if self.embedding_type == "learned":
            self.position_embeddings = nn.Embedding(max_sequence_length, hidden_size, device=dev,
                                                    dtype=neox_args.params_dtype)
            init_method(self.position_embeddings.weight)
        elif self.embedding_type == "sinusoidal":
            self.position_embeddings = SinusoidalPositionalEmbedding(hidden_size, precision=neox_args.params_dtype)
        if num_tokentypes > 0:
            self.tokentype_embeddings = nn.Embedding(num_tokentypes, hidden_size, device=dev,
                                                     dtype=neox_args.params_dtype)
            init_method(self.tokentype_embeddings.weight)
        else:
            self.tokentype_embeddings = None
        self.embedding_dropout = nn.Dropout(embedding_dropout_prob)
        # with 8-bit optimizer states the token embeddings are layer-normalised ("stable embedding")
        self.stable_norm = None
        if getattr(neox_args, "use_bnb_optimizer", False):
            from ..optim.adam8bit import StableEmbeddingNorm
            self.stable_norm = StableEmbeddingNorm(hidden_size, device=dev, dtype=neox_args.params_dtype)
        self.opt_pos_emb_offset = neox_args.opt_pos_emb_offset
        self.layer_past = None

    def add_tokentype_embeddings(self, num_tokentypes):
        if self.tokentype_embeddings is not None:
            raise Exception("tokentype embeddings is already initialized")
        self.num_tokentypes = num_tokentypes
        w = self.word_embeddings.weight
        self.tokentype_embeddings = nn.Embedding(num_tokentypes, self.hidden_size, device=w.device, dtype=w.dtype)
        self.init_method(self.tokentype_embeddings.weight)

    def forward(self, input_ids, position_ids, tokentype_ids=None):
        emb = self.word_embeddings(input_ids)
        if self.stable_norm is not None:
            emb = self.stable_norm(emb)
        if self.embedding_type in ("learned", "sinusoidal"):
            if self.opt_pos_emb_offset:
                if self.layer_past is not None:
                    position_ids = position_ids + self.layer_past + 1
                self.layer_past = position_ids[:, -1]
                position_ids = position_ids + self.opt_pos_emb_offset
            if self.embedding_type == "learned":
                pos = self.position_embeddings(position_ids)
            else:
                pos = self.position_embeddings(input_ids, seq_dim=1).to(emb.dtype)
            emb = emb + pos * self.mup_rp_embedding_mult
        if tokentype_ids is not None:
            assert self.tokentype_embeddings is not None
            emb = emb + self.tokentype_embeddings(tokentype_ids)
        else:
            assert self.tokentype_embeddings is None
        emb = self.embedding_dropout(emb)
        if self.use_mup:
            emb = emb * self.mup_embedding_mult
        if self.sequence_parallel:
            emb = M.scatter_to_sequence_parallel_region(emb, seq_dim=1)
        return emb


class EmbeddingPipe(Embedding):
    """Pipeline form: ``(input_ids, position_ids, attention_mask)`` -> ``(embeddings, attention_mask)``."""

    @property
    def word_embeddings_weight(self):
        return self.word_embeddings.weight

    def forward(self, args):
        assert len(args) == 3, f"Expected 3 arguments (input_ids, position_ids, attention_mask), but got {len(args)}."
        input_ids, position_ids, attention_mask = args
        return super().forward(input_ids, position_ids), attention_mask


class SoftEmbedding(nn.Module):
    """Prompt tuning: ``n_tokens`` trainable vectors prepended to the embedded sequence."""

    def __init__(self, neox_args, wte, n_tokens: int = 10, init_range: float = 0.5, init_string: str = ""):
        super().__init__()
        self.n_tokens, self.neox_args, self.init_range, self.init_string = n_tokens, neox_args, init_range, init_string
        self.soft_embedding_weight = nn.Parameter(self.initialize_embedding(wte))

    def initialize_embedding(self, wte):
        if self.init_string:
            ids = torch.LongTensor(self.neox_args.tokenizer.tokenize(self.init_string)).to(wte.weight.device)
            emb = wte(ids)
            if emb.shape[0] >= self.n_tokens:
                emb = emb[: self.n_tokens, :]
            else:
                emb = emb.repeat(math.ceil(self.n_tokens / emb.shape[0]), 1)[: self.n_tokens, :]
            return emb.detach().clone()
        w = wte.weight
        return torch.empty(self.n_tokens, self.neox_args.hidden_size, device=w.device, dtype=w.dtype).uniform_(
            -self.init_range, self.init_range)

    def forward(self, args: tuple):
        if len(args) == 2:
            embedding, attention_mask = args
            layer_past = None
            training_form = True
        else:
            embedding, layer_past, attention_mask = args
            training_form = False
        soft = self.soft_embedding_weight.repeat(embedding.shape[0], 1, 1)
        if training_form:
            embedding = torch.cat((soft, embedding), dim=1)[:, : self.neox_args.seq_length, ...]
            return embedding, attention_mask
        if not (layer_past is not None and layer_past.numel() > 0):
            embedding = torch.cat((soft, embedding), dim=1)[:, : self.neox_args.seq_length, ...]
        return embedding, layer_past, attention_mask
