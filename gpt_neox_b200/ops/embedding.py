"""Vocabulary-parallel embedding lookup on the kernels of ``csrc/embed_sample.cu``.

``embedding(ids, weight, v0)``: ``weight`` holds vocabulary rows ``[v0, v0 + weight.shape[0])``; ids outside that range
produce zero rows (another tensor-parallel rank owns them and the caller all-reduces).  The backward pass scatter-adds
the gradient rows in fp32 -- straight into ``weight.main_grad`` when the engine provides it -- so no vocabulary-sized
bf16 gradient is materialised.  Reference behaviour: ``megatron/mpu/layers.py:98-180`` (mask, ``F.embedding``,
masked fill).  On CPU or for other dtypes the same math runs through torch ops.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import native
from .linear import main_grad_of


def embedding_ref(ids, weight, v0=0):
    v1 = v0 + weight.shape[0]
    mask = (ids < v0) | (ids >= v1)
    out = F.embedding((ids - v0).masked_fill(mask, 0), weight)
    return out.masked_fill(mask.unsqueeze(-1), 0.0)


class _EmbedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, v0):
        ids_c = ids.contiguous()
        rows, h = weight.shape
        out = torch.empty(*ids.shape, h, dtype=weight.dtype, device=weight.device)
        rc = native.lib().neox_embedding_fwd(native.ptr(ids_c), native.ptr(weight), native.ptr(out),
                                             ctypes.c_longlong(ids_c.numel()), int(h), ctypes.c_longlong(v0),
                                             ctypes.c_longlong(v0 + rows), ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_embedding_fwd")
        ctx.save_for_backward(ids_c)
        ctx.weight, ctx.v0 = weight, v0
        return out

    @staticmethod
    def backward(ctx, g):
        (ids_c,) = ctx.saved_tensors
        weight, v0 = ctx.weight, ctx.v0
        rows, h = weight.shape
        g = g.contiguous()
        mg = main_grad_of(weight)
        target = mg if mg is not None else torch.zeros(rows, h, dtype=torch.float32, device=g.device)
        rc = native.lib().neox_embedding_bwd(native.ptr(ids_c), native.ptr(g), native.ptr(target),
                                             ctypes.c_longlong(ids_c.numel()), int(h), ctypes.c_longlong(v0),
                                             ctypes.c_longlong(v0 + rows), ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_embedding_bwd")
        if mg is not None:
            weight.grad_in_main = True
            from .linear import notify_grad_ready
            notify_grad_ready(weight)
            return None, None, None
        return None, target.to(weight.dtype), None


def kernel_ok(ids, weight) -> bool:
    mg = main_grad_of(weight)
    return (weight.is_cuda and native.available() and weight.dtype == torch.bfloat16 and ids.dtype == torch.int64
            and weight.is_contiguous() and weight.shape[1] % 8 == 0
            and (mg is None or (mg.dtype == torch.float32 and mg.is_contiguous())))


def embedding(ids, weight, v0=0):
    if kernel_ok(ids, weight):
        return _EmbedFn.apply(ids, weight, v0)
    return embedding_ref(ids, weight, v0)
