"""Mixture-of-experts building blocks on the device: fused router, row dispatch / combine, grouped expert GEMMs.

Layout convention: the ``A = T * k`` token-to-expert assignments are stored expert-major in a *padded* activation
matrix -- expert ``e`` owns the rows ``[start_e, start_e + count_e)`` with ``start_e = sum_{i<e} round_up(count_i,
PAD)``; padding rows hold zeros.  ``PAD = 64`` is the contraction block of the grouped weight-gradient GEMM.  The
matrix has a static number of rows (``padded_rows``), so nothing downstream of the router depends on a value the
host would have to read back: no synchronisation between routing and the expert GEMMs.

Kernels: ``csrc/moe_kernels.cu`` (router forward / backward, dispatch, combine) and the grouped modes of the tcgen05
GEMM in ``csrc/gemm_sm100.cu``.  Every function has an eager fp32 statement (``*_ref``) used on CPU and as the
oracle of the GPU tests.  Reference counterparts: ``megatron/model/router.py`` (top-k router), ``megatron/model/
moe_mlp.py`` (grouped expert MLP through MegaBlocks' ``gmm``), ``megatron/model/moe.py`` (permute / un-permute).
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import flop_count, native
from . import gemm as G
from .functional import _DT, dgelu_mul
from .linear import main_grad_of

PAD = 64


def padded_rows(assignments: int, experts: int) -> int:
    """Static row count of the padded expert-major matrix for that many assignments."""
    return (assignments + experts * (PAD - 1) + 127) // 128 * 128


def _s():
    return ctypes.c_void_p(native.stream_ptr())


# ------------------------------------------------------------------------------------------------ router
def router_ref(logits, k):
    probs = F.softmax(logits.float(), dim=-1)
    w, idx = torch.topk(probs, k, dim=-1)
    if k > 1:
        w = w / w.sum(dim=-1, keepdim=True)
    counts = torch.bincount(idx.reshape(-1), minlength=logits.shape[-1])
    return probs, w, idx, counts


def router_kernel_ok(logits, k):
    return logits.is_cuda and native.available() and logits.dtype in _DT and logits.shape[-1] <= 512 and k <= 8


class _RouterFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, k):
        T, E = logits.shape
        logits = logits.contiguous()
        probs = torch.empty(T, E, dtype=torch.float32, device=logits.device)
        w = torch.empty(T, k, dtype=torch.float32, device=logits.device)
        idx = torch.empty(T, k, dtype=torch.int64, device=logits.device)
        counts = torch.zeros(E, dtype=torch.int64, device=logits.device)
        rc = native.lib().neox_moe_router_fwd(native.ptr(logits), native.ptr(probs), native.ptr(w), native.ptr(idx),
                                              native.ptr(counts), T, E, k, _DT[logits.dtype], _s())
        native.check(rc, "neox_moe_router_fwd")
        ctx.save_for_backward(probs, w, idx)
        ctx.k, ctx.dtype = k, logits.dtype
        ctx.mark_non_differentiable(idx, counts)
        return probs, w, idx, counts

    @staticmethod
    def backward(ctx, dprobs, dw, _i, _c):
        probs, w, idx = ctx.saved_tensors
        T, E = probs.shape
        dlogits = torch.empty(T, E, dtype=ctx.dtype, device=probs.device)
        dprobs = dprobs.float().contiguous() if dprobs is not None else None
        dw = dw.float().contiguous() if dw is not None else None
        rc = native.lib().neox_moe_router_bwd(native.ptr(probs), native.ptr(w), native.ptr(idx), native.ptr(dw),
                                              native.ptr(dprobs), native.ptr(dlogits), T, E, ctx.k, _DT[ctx.dtype], _s())
        native.check(rc, "neox_moe_router_bwd")
        return dlogits, None


def router(logits, k):
    """``(probs [T, E] fp32, weights [T, k] fp32 (renormalised for k > 1), experts [T, k] int64, counts [E] int64)``."""
    if router_kernel_ok(logits, k):
        return _RouterFn.apply(logits, k)
    return router_ref(logits, k)


# ------------------------------------------------------------------------------------------------ row plan
def plan_rows(idx, counts, capacity=None):
    """Row of the padded expert-major matrix for every assignment (``[T, k]`` int64, ``-1`` for assignments beyond
    an expert's ``capacity``), and the per-expert counts after the capacity clamp.  Token order is kept inside an
    expert.  Device-side tensor ops only."""
    T, k = idx.shape
    A = T * k
    flat = idx.reshape(-1)
    order = torch.argsort(flat, stable=True)
    sorted_e = flat[order]
    starts = torch.cumsum(counts, 0) - counts
    pos = torch.arange(A, device=idx.device) - starts[sorted_e]
    kept = counts if capacity is None else torch.clamp(counts, max=capacity)
    padded = (kept + (PAD - 1)) // PAD * PAD
    pstarts = torch.cumsum(padded, 0) - padded
    dst = pstarts[sorted_e] + pos
    if capacity is not None:
        dst = torch.where(pos < capacity, dst, torch.full_like(dst, -1))
    row_of = torch.empty_like(dst)
    row_of[order] = dst
    return row_of.view(T, k), kept


# ------------------------------------------------------------------------------------------------ dispatch / combine
def _rows_kernel_ok(x):
    return x.is_cuda and native.available() and x.dtype in (torch.bfloat16, torch.float16) and x.shape[-1] % 8 == 0


def dispatch_ref(x, row_of, rows, scale=None):
    T, k = row_of.shape
    out = torch.zeros(rows, x.shape[1], dtype=x.dtype, device=x.device)
    flat = row_of.reshape(-1)
    ok = flat >= 0
    src = x.repeat_interleave(k, dim=0)
    if scale is not None:
        src = (src.float() * scale.reshape(-1, 1).float()).to(x.dtype)
    out[flat[ok]] = src[ok]
    return out


def combine_ref(src, row_of, gate=None):
    T, k = row_of.shape
    rows = src[row_of.clamp(min=0).reshape(-1)].float().view(T, k, -1)
    wgt = (row_of >= 0).float() if gate is None else gate.float() * (row_of >= 0).float()
    return (rows * wgt.unsqueeze(-1)).sum(1).to(src.dtype)


def _dispatch(x, row_of, rows, scale=None, other=None):
    T, k = row_of.shape
    out = torch.zeros(rows, x.shape[1], dtype=x.dtype, device=x.device)
    dots = torch.empty(T, k, dtype=torch.float32, device=x.device) if other is not None else None
    rc = native.lib().neox_moe_dispatch(native.ptr(x), native.ptr(row_of), native.ptr(scale), native.ptr(out),
                                        native.ptr(other), native.ptr(dots), ctypes.c_longlong(T), k, x.shape[1],
                                        _DT[x.dtype], _s())
    native.check(rc, "neox_moe_dispatch")
    return out, dots


def _combine(src, row_of, gate=None):
    T, k = row_of.shape
    y = torch.empty(T, src.shape[1], dtype=src.dtype, device=src.device)
    rc = native.lib().neox_moe_combine(native.ptr(src), native.ptr(row_of), native.ptr(gate), native.ptr(y),
                                       ctypes.c_longlong(T), k, src.shape[1], _DT[src.dtype], _s())
    native.check(rc, "neox_moe_combine")
    return y


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, row_of, rows):
        ctx.save_for_backward(row_of)
        return _dispatch(x.contiguous(), row_of, rows)[0]

    @staticmethod
    def backward(ctx, g):
        (row_of,) = ctx.saved_tensors
        return _combine(g.contiguous(), row_of), None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, row_of, gate):
        ctx.save_for_backward(src, row_of, gate)
        return _combine(src, row_of, gate)

    @staticmethod
    def backward(ctx, dy):
        src, row_of, gate = ctx.saved_tensors
        d_src, d_gate = _dispatch(dy.contiguous(), row_of, src.shape[0], scale=gate, other=src)
        return d_src, None, d_gate


def dispatch(x, row_of, rows):
    """Copy token rows into the padded expert-major matrix (``rows`` rows, zeros elsewhere)."""
    if _rows_kernel_ok(x):
        return _DispatchFn.apply(x, row_of.contiguous(), rows)
    return dispatch_ref(x, row_of, rows)


def combine(src, row_of, gate):
    """``y[t] = sum_j gate[t, j] * src[row_of[t, j]]`` (fp32 gates, fixed summation order)."""
    if _rows_kernel_ok(src):
        return _CombineFn.apply(src.contiguous(), row_of.contiguous(), gate.float().contiguous())
    return combine_ref(src, row_of, gate)


# ------------------------------------------------------------------------------------------------ grouped GEMM
def _segments(counts):
    c = counts.tolist()
    out, row = [], 0
    for n in c:
        out.append((row, n))
        row += (n + PAD - 1) // PAD * PAD
    return out


def grouped_linear_ref(x_pad, w, counts, act=None):
    """Eager statement: rows of segment e times ``w[e].T`` (padding rows and the rows behind the last segment give
    zeros, as in the kernel, which runs them -- all-zero inputs -- through the GEMM as well)."""
    out = torch.zeros(x_pad.shape[0], w.shape[1], dtype=x_pad.dtype, device=x_pad.device)
    for e, (row, n) in enumerate(_segments(counts)):
        if n:
            flop_count.gemm(n, w.shape[1], w.shape[2])
            y = x_pad[row:row + n] @ w[e].t()
            out[row:row + n] = F.gelu(y, approximate="tanh") if act == "gelu" else y
    return out


def _grouped_call(A, B, D, M, N, K, lda, ldb, ldd, b_mn, counts, E, mode, add=None, preact=None, act=G.ACT_NONE):
    num_n = (N + 255) // 256
    max_tiles = (M // 128 + E + 1) * num_n if mode == 1 else E * ((M + 127) // 128) * num_n
    table = torch.empty(max_tiles * 4 + 4, dtype=torch.int32, device=A.device)   # [ntiles, pad x 3, entries]
    ll = ctypes.c_longlong
    rc = native.lib().neox_gemm_grouped_16(
        native.ptr(A), native.ptr(B), native.ptr(D), M, N, K, ll(lda), ll(ldb), ll(ldd), int(b_mn),
        int(D.dtype == torch.float32), native.ptr(add), ll(add.stride(0) if add is not None else 0),
        int(add is not None and add.dtype == torch.float32), native.ptr(preact),
        ll(preact.stride(0) if preact is not None else 0), None, ll(0), int(act), ctypes.c_float(1.0),
        native.ptr(counts), E, PAD, mode, ctypes.c_void_p(table.data_ptr() + 16), max_tiles,
        ctypes.c_void_p(table.data_ptr()), int(A.dtype == torch.float16), _s())
    native.check(rc, "neox_gemm_grouped_16")


def grouped_kernel_ok(x_pad, w):
    E, N, K = w.shape
    return (x_pad.is_cuda and native.available() and x_pad.dtype in (torch.bfloat16, torch.float16)
            and w.dtype == x_pad.dtype and w.is_contiguous() and x_pad.is_contiguous() and x_pad.shape[0] % 128 == 0
            and N % 64 == 0 and K % 64 == 0 and E <= 4096)


class _GroupedLinearFn(torch.autograd.Function):
    """``y[rows of e] = act(x[rows of e] @ w[e].T)`` for all experts in one launch; dgrad in one launch (weights read
    MN-major), wgrad in one launch (contraction over each expert's own rows, accumulated into ``main_grad`` when the
    optimizer provides it)."""

    @staticmethod
    def forward(ctx, x_pad, w, counts, act):
        E, N, K = w.shape
        M = x_pad.shape[0]
        flop_count.gemm(M, N, K)
        out = torch.empty(M, N, dtype=x_pad.dtype, device=x_pad.device)
        pre = torch.empty_like(out) if act == "gelu" else None
        _grouped_call(x_pad, w, out, M, N, K, K, K, N, False, counts, E, 1, preact=pre,
                      act=G.ACT_GELU if act == "gelu" else G.ACT_NONE)
        ctx.save_for_backward(x_pad, w, counts, pre)
        ctx.act = act
        return out

    @staticmethod
    def backward(ctx, g):
        x_pad, w, counts, pre = ctx.saved_tensors
        E, N, K = w.shape
        M = x_pad.shape[0]
        g = g.contiguous()
        if ctx.act == "gelu":
            g = dgelu_mul(g, pre)
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = torch.empty(M, K, dtype=x_pad.dtype, device=x_pad.device)
            # the stacked weights [E * N, K] read MN-major: contraction over N, expert e at contraction rows e * N
            _grouped_call(g, w, gx, M, K, N, N, K, K, True, counts, E, 1)
        if ctx.needs_input_grad[1]:
            mg = main_grad_of(w)
            if mg is not None:
                _grouped_call(g, x_pad, mg.view(E * N, K), N, K, M, N, K, K, True, counts, E, 2, add=mg.view(E * N, K))
                w.grad_in_main = True
                from .linear import notify_grad_ready
                notify_grad_ready(w)
            else:
                gw = torch.zeros(E, N, K, dtype=w.dtype, device=w.device)    # experts without tokens keep zeros
                _grouped_call(g, x_pad, gw.view(E * N, K), N, K, M, N, K, K, True, counts, E, 2)
        return gx, gw, None, None


def grouped_linear(x_pad, w, counts, act=None):
    """Expert linear layers over the padded expert-major matrix: ``w`` is ``[E, out, in]``, ``counts`` the int64
    per-expert row counts on the device, ``act`` ``None`` or ``"gelu"`` (fused into the GEMM epilogue)."""
    if grouped_kernel_ok(x_pad, w):
        return _GroupedLinearFn.apply(x_pad, w, counts.contiguous(), act)
    return grouped_linear_ref(x_pad, w, counts, act)
