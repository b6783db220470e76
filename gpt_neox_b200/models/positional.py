"""Positional information: rotary, ALiBi and sinusoidal
(reference ``megatron/model/positional_embeddings.py:19-257``)."""
from __future__ import annotations

import math

import torch
import torch.nn as nn

from ..ops import functional as OF


class SinusoidalPositionalEmbedding(nn.Module):
    def __init__(self, dim, base=10000, precision=torch.half):
        super().__init__()
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
        self.register_buffer("inv_freq", inv_freq)
        self.precision = precision

    def forward(self, x, seq_dim=1):
        t = torch.arange(x.shape[seq_dim], device=x.device).type_as(self.inv_freq)
        sinusoid = torch.einsum("i,j->ij", t, self.inv_freq.to(x.device))
        emb = torch.cat((sinusoid.sin(), sinusoid.cos()), dim=-1)
        return emb[None, :, :].to(self.precision if x.is_cuda else torch.float32)


class RotaryEmbedding(nn.Module):
    """Pre-computed cos/sin tables ``[max_seq, 1, 1, dim]`` in fp32; ``forward`` returns views."""

    def __init__(self, dim, max_seq_len, base=10000, precision=torch.half, save_inv_freqs=False):
        super().__init__()
        inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2).float() / dim))
        self.register_buffer("inv_freq", inv_freq, persistent=save_inv_freqs)
        self.dim, self.base, self.max_seq_len, self.precision = dim, base, max_seq_len, precision
        cos, sin = self._tables(max_seq_len, inv_freq.device)
        self.register_buffer("cos_cached", cos, persistent=False)
        self.register_buffer("sin_cached", sin, persistent=False)

    def _tables(self, seq_len, device):
        t = torch.arange(seq_len, device=device).float()
        inv = 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=device).float() / self.dim))
        freqs = torch.einsum("i,j->ij", t, inv)
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos()[:, None, None, :], emb.sin()[:, None, None, :]

    def forward(self, x, seq_dim=0, seq_len=None):
        if seq_len is None:
            seq_len = x.shape[seq_dim]
        assert seq_len <= self.max_seq_len, f"sequence length {seq_len} exceeds rotary table ({self.max_seq_len})"
        if self.cos_cached.device != x.device:
            self.cos_cached, self.sin_cached = self.cos_cached.to(x.device), self.sin_cached.to(x.device)
        return self.cos_cached[:seq_len], self.sin_cached[:seq_len]


def apply_rotary_pos_emb(q, k, cos, sin, offset: int = 0):
    """q, k: [s, b, h, rot]; tables are sliced at ``offset`` (kv-cache decoding)."""
    cos_q, sin_q = cos[offset:q.shape[0] + offset], sin[offset:q.shape[0] + offset]
    return OF.rope(q, cos_q, sin_q), OF.rope(k, cos_q, sin_q)


class AliBi(nn.Module):
    """Linear attention biases; slopes are sharded by tensor-parallel rank."""

    def __init__(self, num_heads, mp_size=1, mp_rank=0):
        super().__init__()
        assert mp_size <= num_heads and mp_rank <= mp_size
        self.mp_size, self.mp_rank, self.num_heads = mp_size, mp_rank, num_heads
        self.slice_size = num_heads // mp_size
        self.cached_matrix, self.cached_seq_len = None, None
        slopes = torch.tensor(self._get_slopes(num_heads))[mp_rank * self.slice_size:(mp_rank + 1) * self.slice_size]
        self.register_buffer("slopes", slopes)

    @staticmethod
    def _get_slopes(n):
        def pow2(n):
            start = 2 ** (-(2 ** -(math.log2(n) - 3)))
            return [start * start ** i for i in range(n)]
        if math.log2(n).is_integer():
            return pow2(n)
        closest = 2 ** math.floor(math.log2(n))
        return pow2(closest) + AliBi._get_slopes(2 * closest)[0::2][: n - closest]

    def bias(self, seq_len_q, seq_len_k, device, dtype):
        target = max(seq_len_q, seq_len_k)
        if self.cached_seq_len is not None and self.cached_seq_len >= target and self.cached_matrix.device == device:
            a = self.cached_matrix[:target, :target]
        else:
            a = -torch.tril(torch.arange(target).view(target, 1).repeat(1, target)
                            + torch.arange(0, -target, -1)).to(device).float()
            self.cached_seq_len, self.cached_matrix = target, a
        if seq_len_q != seq_len_k:
            a = a[seq_len_k - seq_len_q:, :] if seq_len_q != 1 else a[seq_len_k - 1:seq_len_k, :]
        a = a[:seq_len_q, :seq_len_k]
        return (a[None] * self.slopes.to(device).float().view(-1, 1, 1)).to(dtype)

    def forward(self, x):
        # x: [b, np, sq, sk]
        return x + self.bias(x.shape[-2], x.shape[-1], x.device, x.dtype)
