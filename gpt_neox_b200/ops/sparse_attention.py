"""Block-sparse causal attention that only touches the blocks of the layout.

The reference's sparse attention types (``megatron/model/utils.py:253-353``: ``local``, ``sparse_fixed``,
``sparse_variable``, ``bigbird``, ``bslongformer``) run on DeepSpeed's Triton block-sparse matmul / softmax.  Here the
layout is a boolean matrix over ``block x block`` tiles of the score matrix; for every query block the key / value
blocks it may attend to are gathered (padded to the largest count of any row), and scores, softmax and the weighted
sum are computed on that ``[query block, kept key blocks]`` slab only: ``O(s * kept * block * d)`` work and memory
instead of the ``O(s^2 d)`` of masking a dense score matrix.  The batched matmuls go to the library GEMM; everything
is plain autograd, so the backward is sparse too.  ``models/transformer.py::sparse_layout_mask`` stays as the dense
statement of the same layouts (the test oracle, and the path taken with a key/value cache).
"""
from __future__ import annotations

import torch

_PLANS = {}


def block_layout(kind, nq, nk, cfg):
    """Boolean ``[nq, nk]`` matrix (True = the tile is computed) of one layout, before the causal cut."""
    qi = torch.arange(nq)[:, None]
    ki = torch.arange(nk)[None, :]
    if kind == "local":
        w = int(cfg.get("num_sliding_window_blocks", 3))
        keep = (qi - ki).abs() <= w // 2
    elif kind in ("sparse_fixed", "sparse_variable"):
        local = int(cfg.get("num_local_blocks", 4))
        nglob = int(cfg.get("num_global_blocks", 1))
        keep = (qi // local) == (ki // local)
        keep = keep | ((ki % local) >= (local - nglob))
    elif kind == "bigbird":
        w = int(cfg.get("num_sliding_window_blocks", 3))
        nglob = int(cfg.get("num_global_blocks", 1))
        nrand = int(cfg.get("num_random_blocks", 1))
        keep = ((qi - ki).abs() <= w // 2) | (ki < nglob) | (qi < nglob)
        g = torch.Generator().manual_seed(0)
        rnd = torch.rand(nq, nk, generator=g)
        keep = keep | (rnd >= torch.topk(rnd, min(nrand, nk), dim=-1).values[:, -1:])
    elif kind == "bslongformer":
        w = int(cfg.get("num_sliding_window_blocks", 3))
        keep = (qi - ki).abs() <= w // 2
        for gidx in cfg.get("global_block_indices", [0]):
            keep = keep | (ki == gidx) | (qi == gidx)
    else:
        raise ValueError(f"unknown sparse attention type {kind}")
    return keep


def _plan(kind, s, block, cfg, device):
    """Per query block: indices of the kept key blocks (padded with 0) and which of them are real."""
    key = (kind, s, block, tuple(sorted((k, str(v)) for k, v in cfg.items())), str(device))
    plan = _PLANS.get(key)
    if plan is None:
        n = (s + block - 1) // block
        keep = block_layout(kind, n, n, cfg) & (torch.arange(n)[None, :] <= torch.arange(n)[:, None])   # causal cut
        counts = keep.sum(1)
        kmax = int(counts.max())
        order = torch.argsort((~keep).to(torch.int8), dim=1, stable=True)[:, :kmax]      # kept blocks first, ascending
        valid = torch.arange(kmax)[None, :] < counts[:, None]
        order = torch.where(valid, order, torch.zeros_like(order))
        plan = (order.to(device), valid.to(device), n, kmax)
        _PLANS[key] = plan
    return plan


def block_sparse_attention(q, k, v, kind, cfg, scale, dropout=None):
    """``q, k, v``: ``[s, b, heads, d]`` (same ``s``; key/value heads may be fewer: grouped-query).  Causal.
    ``dropout``: optional callable applied to the probabilities.  Returns ``[s, b, heads, d]``."""
    s, b, h, d = q.shape
    block = int(cfg.get("block", 16))
    if k.shape[2] != h:
        rep = h // k.shape[2]
        k = k.repeat_interleave(rep, dim=2)
        v = v.repeat_interleave(rep, dim=2)
    order, valid, n, kmax = _plan(kind, s, block, cfg, q.device)
    pad = n * block - s

    def blocks(t):
        t = t.permute(1, 2, 0, 3)                                   # [b, h, s, d]
        if pad:
            t = torch.nn.functional.pad(t, (0, 0, 0, pad))
        return t.reshape(b, h, n, block, d)
    qb, kb, vb = blocks(q), blocks(k), blocks(v)
    kg = kb[:, :, order]                                            # [b, h, n, kmax, block, d]
    vg = vb[:, :, order]
    scores = torch.einsum("bhqid,bhqmjd->bhqimj", qb, kg).float() * scale
    # key position of every gathered column, query position of every row: causal inside and across tiles, padding off
    kpos = order[:, :, None] * block + torch.arange(block, device=q.device)[None, None, :]          # [n, kmax, block]
    qpos = torch.arange(n, device=q.device)[:, None] * block + torch.arange(block, device=q.device)[None, :]  # [n, block]
    dead = (~valid)[:, None, :, None] | (kpos[:, None] > qpos[:, :, None, None]) | (kpos[:, None] >= s)
    scores = scores.masked_fill(dead[None, None], float("-inf"))
    flat = scores.reshape(b, h, n, block, kmax * block)
    probs = torch.softmax(flat, dim=-1)
    probs = torch.nan_to_num(probs, nan=0.0)                       # padded query rows have no live column
    probs = probs.to(q.dtype)
    if dropout is not None:
        probs = dropout(probs)
    out = torch.einsum("bhqimj,bhqmjd->bhqid", probs.reshape(b, h, n, block, kmax, block), vg)
    out = out.reshape(b, h, n * block, d)[:, :, :s]
    return out.permute(2, 0, 1, 3).contiguous()
