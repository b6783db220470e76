"""Fused multi-head attention (flash attention) front-end.

``flash_attention(q, k, v)`` takes the ``[s, b, heads, d]`` views the transformer layer slices out of
the fused QKV projection -- without making them contiguous -- and returns ``[sq, b, heads, d]``.
Supported: causal masking (bottom-right aligned when ``sq < sk``, as needed for kv-cache decoding),
sliding windows, ALiBi slopes, grouped-query attention (``heads_q % heads_kv == 0``), head sizes
64 / 96 / 128 on the sm_100a kernel (``csrc/flash_attn_sm100.cu``: QK^T and PV on tcgen05 with S and
O accumulators in tensor memory).  Reference: the flash-attn 2 calls in
``megatron/model/transformer.py:627-744``.

``attention_ref`` is the fp32 statement of the same math (CPU path and test oracle).
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import flop_count, native
from .functional import _DT, _s


def attention_ref(q, k, v, causal=True, softmax_scale=None, window=None, alibi_slopes=None, bias=None,
                  return_lse=False):
    sq, b, hq, d = q.shape
    sk, _, hkv, _ = k.shape
    flop_count.attention(b, hq, sq, sk, d, causal)
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    qf = q.float().permute(1, 2, 0, 3)                       # [b, hq, sq, d]
    kf = k.float().permute(1, 2, 0, 3)
    vf = v.float().permute(1, 2, 0, 3)
    if hkv != hq:
        rep = hq // hkv
        kf = kf.repeat_interleave(rep, dim=1)
        vf = vf.repeat_interleave(rep, dim=1)
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale  # [b, hq, sq, sk]
    qi = torch.arange(sq, device=q.device)[:, None] + (sk - sq)
    ki = torch.arange(sk, device=q.device)[None, :]
    if alibi_slopes is not None:
        scores = scores + (-(qi - ki).abs().float())[None, None] * alibi_slopes.float().view(1, -1, 1, 1)
    if bias is not None:
        scores = scores + bias.float()
    mask = torch.zeros(sq, sk, dtype=torch.bool, device=q.device)
    if causal:
        mask |= ki > qi
    if window is not None:
        mask |= ki < qi - window
    scores = scores.masked_fill(mask[None, None], float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)
    p = torch.softmax(scores, dim=-1)
    out = torch.matmul(p, vf).permute(2, 0, 1, 3).contiguous().to(q.dtype)
    return (out, lse) if return_lse else out


def kernel_ok(q, k, v, bias=None) -> bool:
    if not (q.is_cuda and native.available()):
        return False
    ok = (q.dtype in (torch.bfloat16, torch.float16) and k.dtype == q.dtype and v.dtype == q.dtype and bias is None
          and q.shape[-1] in (64, 96, 128) and q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1
          and q.shape[0] >= 1)
    if not ok:
        from .linear import warn_fallback
        warn_fallback("flash_attention", f"dtype {q.dtype}, head size {q.shape[-1]}, additive bias {bias is not None}")
    return ok


def _launch_fwd(q, k, v, out, lse, sq, sk, b, hq, hkv, d, scale, causal, window, slopes):
    """Forward kernel launch.  Default: the two-query-tile kernel (``csrc/flash_fwd2_sm100.cu``, P kept in tensor
    memory); ``NEOX_FLASH_FWD=1`` selects the one-tile kernel (``csrc/flash_fwd_sm100.cu``, bf16 only)."""
    L = native.lib()
    ll = ctypes.c_longlong
    strides = (ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)),
               ll(v.stride(0)), ll(v.stride(1)), ll(v.stride(2)))
    tail = (ctypes.c_float(scale), int(causal), int(window if window is not None else -1), native.ptr(slopes))
    if os.environ.get("NEOX_FLASH_FWD", "2") == "1" and q.dtype == torch.bfloat16:
        rc = L.neox_flash_fwd(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(out), native.ptr(lse),
                              sq, sk, b, hq, hkv, d, *strides, *tail, _s())
        native.check(rc, "neox_flash_fwd")
        return
    rc = L.neox_flash_fwd2(native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(out), native.ptr(lse),
                           sq, sk, b, hq, hkv, d, *strides, *tail, _DT[q.dtype], _s())
    native.check(rc, "neox_flash_fwd2")


def _launch_bwd(q, k, v, out, do, lse, dq, dk, dv, delta, gs, sq, sk, b, hq, hkv, d, scale, causal, window, slopes):
    """Backward kernels (delta, dK/dV, dQ) writing into the strided ``dq`` / ``dk`` / ``dv`` views (``gs``: their
    nine element strides).  Default: 128-wide blocks with P / dS kept in tensor memory
    (``csrc/flash_bwd2_sm100.cu``); ``NEOX_FLASH_BWD=1`` selects the 64-wide form (``csrc/flash_bwd_sm100.cu``)."""
    L = native.lib()
    ll = ctypes.c_longlong
    args = (native.ptr(q), native.ptr(k), native.ptr(v), native.ptr(out), native.ptr(do), native.ptr(lse),
            native.ptr(dq), native.ptr(dk), native.ptr(dv), native.ptr(delta), sq, sk, b, hq, hkv, d,
            ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)), ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)),
            ll(v.stride(0)), ll(v.stride(1)), ll(v.stride(2)), gs,
            ctypes.c_float(scale), int(causal), int(window if window is not None else -1), native.ptr(slopes))
    if os.environ.get("NEOX_FLASH_BWD", "2") == "1" and q.dtype == torch.bfloat16:
        native.check(L.neox_flash_bwd_strided(*args, _s()), "neox_flash_bwd_strided")
    else:
        native.check(L.neox_flash_bwd2_strided(*args, _DT[q.dtype], _s()), "neox_flash_bwd2_strided")


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, causal, scale, window, slopes):
        sq, b, hq, d = q.shape
        sk, _, hkv, _ = k.shape
        out = torch.empty(sq, b, hq, d, dtype=q.dtype, device=q.device)
        lse = torch.empty(b, hq, sq, dtype=torch.float32, device=q.device)
        flop_count.attention(b, hq, sq, sk, d, causal)
        _launch_fwd(q, k, v, out, lse, sq, sk, b, hq, hkv, d, scale, causal, window, slopes)
        ctx.save_for_backward(q, k, v, out, lse, slopes if slopes is not None else torch.empty(0, device=q.device))
        ctx.cfg = (causal, scale, window, slopes is not None)
        return out

    @staticmethod
    def backward(ctx, do):
        q, k, v, out, lse, slopes = ctx.saved_tensors
        causal, scale, window, has_slopes = ctx.cfg
        sq, b, hq, d = q.shape
        sk, _, hkv, _ = k.shape
        do = do.contiguous()
        dq = torch.empty(sq, b, hq, d, dtype=q.dtype, device=q.device)
        dk = torch.empty(sk, b, hkv, d, dtype=q.dtype, device=q.device)
        dv = torch.empty(sk, b, hkv, d, dtype=q.dtype, device=q.device)
        delta = torch.empty(b, hq, sq, dtype=torch.float32, device=q.device)
        L = native.lib()
        ll = ctypes.c_longlong
        gs = (ctypes.c_longlong * 9)(dq.stride(0), dq.stride(1), dq.stride(2), dk.stride(0), dk.stride(1), dk.stride(2),
                                     dv.stride(0), dv.stride(1), dv.stride(2))
        _launch_bwd(q, k, v, out, do, lse, dq, dk, dv, delta, gs, sq, sk, b, hq, hkv, d, scale, causal, window,
                    slopes if has_slopes else None)
        return dq, dk, dv, None, None, None, None


class _PackedQKVFn(torch.autograd.Function):
    """Rotary embedding + causal flash attention on the packed projection ``mixed`` = [s, b, heads, 3 * d]
    (q | k | v per head), entirely in place:

    * forward rotates the first ``rot`` dims of q and k INSIDE ``mixed`` (its producer, the QKV GEMM, does not need
      its own output again) and runs the attention kernel on the three strided views;
    * backward lets the attention kernels write dq / dk / dv straight into the three views of one ``d_mixed``
      buffer and un-rotates dq and dk there, so the gradient of the projection is born packed.

    Compared with slicing + out-of-place rotary this removes two full-tensor rotary passes, the three zero-filled
    slice gradients and their adds, and the contiguous copies in front of the QKV weight-gradient GEMM.
    """

    @staticmethod
    def forward(ctx, mixed, cos, sin, causal, scale, window, slopes):
        s, b, h, d3 = mixed.shape
        d = d3 // 3
        assert mixed.is_contiguous()
        flop_count.attention(b, h, s, s, d, causal)
        q, k, v = mixed[..., :d], mixed[..., d:2 * d], mixed[..., 2 * d:]
        L = native.lib()
        ll = ctypes.c_longlong
        rot = 0
        c = sn = None
        if cos is not None:
            rot = cos.shape[-1]
            c = cos.reshape(-1, rot)[:s].float().contiguous()
            sn = sin.reshape(-1, rot)[:s].float().contiguous()
            rc = L.neox_rope_qk_inplace(native.ptr(q), native.ptr(k), native.ptr(c), native.ptr(sn), s, b, h, h, rot,
                                        ll(q.stride(0)), ll(q.stride(1)), ll(q.stride(2)),
                                        ll(k.stride(0)), ll(k.stride(1)), ll(k.stride(2)), 0, _DT[mixed.dtype], _s())
            native.check(rc, "neox_rope_qk_inplace")
        out = torch.empty(s, b, h, d, dtype=mixed.dtype, device=mixed.device)
        lse = torch.empty(b, h, s, dtype=torch.float32, device=mixed.device)
        _launch_fwd(q, k, v, out, lse, s, s, b, h, h, d, scale, causal, window, slopes)
        empty = torch.empty(0, device=mixed.device)
        ctx.save_for_backward(mixed, out, lse, slopes if slopes is not None else empty,
                              c if c is not None else empty, sn if sn is not None else empty)
        ctx.cfg = (causal, scale, window, slopes is not None, rot)
        return out

    @staticmethod
    def backward(ctx, do):
        mixed, out, lse, slopes, c, sn = ctx.saved_tensors
        causal, scale, window, has_slopes, rot = ctx.cfg
        s, b, h, d3 = mixed.shape
        d = d3 // 3
        q, k, v = mixed[..., :d], mixed[..., d:2 * d], mixed[..., 2 * d:]
        do = do.contiguous()
        dm = torch.empty_like(mixed)
        dq, dk, dv = dm[..., :d], dm[..., d:2 * d], dm[..., 2 * d:]
        delta = torch.empty(b, h, s, dtype=torch.float32, device=mixed.device)
        L = native.lib()
        ll = ctypes.c_longlong
        gs = (ctypes.c_longlong * 9)(dq.stride(0), dq.stride(1), dq.stride(2), dk.stride(0), dk.stride(1), dk.stride(2),
                                     dv.stride(0), dv.stride(1), dv.stride(2))
        _launch_bwd(q, k, v, out, do, lse, dq, dk, dv, delta, gs, s, s, b, h, h, d, scale, causal, window,
                    slopes if has_slopes else None)
        if rot:
            rc = L.neox_rope_qk_inplace(native.ptr(dq), native.ptr(dk), native.ptr(c), native.ptr(sn), s, b, h, h, rot,
                                        ll(dq.stride(0)), ll(dq.stride(1)), ll(dq.stride(2)),
                                        ll(dk.stride(0)), ll(dk.stride(1)), ll(dk.stride(2)), 1, _DT[mixed.dtype], _s())
            native.check(rc, "neox_rope_qk_inplace")
        return dm, None, None, None, None, None, None


def packed_qkv_ok(mixed, head_dim) -> bool:
    return (mixed.is_cuda and native.available() and mixed.dtype in (torch.bfloat16, torch.float16) and mixed.dim() == 4
            and mixed.is_contiguous() and head_dim in (64, 96, 128) and mixed.shape[-1] == 3 * head_dim
            and have_flash_kernel())


def packed_qkv_attention(mixed, cos=None, sin=None, causal=True, softmax_scale=None, window=None, alibi_slopes=None):
    """``flash_attention(rope(q), rope(k), v)`` for ``mixed`` = [s, b, heads, 3 * d]; ``mixed`` is overwritten.
    ``cos`` / ``sin``: [s, 1, 1, rot] tables (None = no rotary)."""
    d = mixed.shape[-1] // 3
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    slopes = alibi_slopes.float().contiguous() if alibi_slopes is not None else None
    return _PackedQKVFn.apply(mixed, cos, sin, causal, scale, window, slopes)


_FLASH_IMPL = {"fwd": None}


def have_flash_kernel() -> bool:
    if _FLASH_IMPL["fwd"] is None:
        _FLASH_IMPL["fwd"] = native.lib().has("neox_flash_fwd") if native.available() else False
    return _FLASH_IMPL["fwd"]


def flash_attention(q, k, v, causal=True, softmax_scale=None, window=None, alibi_slopes=None, bias=None):
    d = q.shape[-1]
    scale = softmax_scale if softmax_scale is not None else 1.0 / math.sqrt(d)
    if kernel_ok(q, k, v, bias) and have_flash_kernel():
        slopes = alibi_slopes.float().contiguous() if alibi_slopes is not None else None
        return _FlashFn.apply(q, k, v, causal, scale, window, slopes)
    return attention_ref(q, k, v, causal, scale, window, alibi_slopes, bias)
