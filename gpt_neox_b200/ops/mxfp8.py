"""Block-scaled FP8 (MXFP8) tensors and the linear layer that trains through them.

Format (OCP microscaling): blocks of 32 elements along the contraction dimension share one power-of-two scale
(E8M0 byte); elements are FP8 -- E4M3 for activations and weights, E5M2 for gradients under the ``hybrid`` format
(``te_fp8_format``), E4M3 everywhere under ``e4m3``.  ``quantize`` / ``dequantize`` expose the storage form
(bytes + scales); ``qdq`` is the fused round trip the linear layer uses.

``mx_linear``: every GEMM of the layer -- forward ``x W^T``, data gradient ``dy W`` and weight gradient ``dy^T x`` --
takes both operands quantised in 32-blocks along ITS contraction dimension (hidden, output features and tokens
respectively), as a hardware block-scaled MMA would.  Because an FP8 value times a power of two is exact in bf16,
running the bf16 tcgen05 GEMM (fp32 accumulation) on the dequantised operands yields exactly the block-scaled
products; the fp8 tensor-core rate is not reached on this path.  This is the behaviour behind the ``te_columnparallel``
/ ``te_rowparallel`` switches (reference: ``megatron/model/transformer_engine.py``, which wraps Transformer Engine's
delayed-scaling fp8 layers; block scaling needs no amax history, so the ``te_fp8_amax_*`` keys are accepted and unused).
"""
from __future__ import annotations

import ctypes

import torch

from . import gemm as G
from . import native
from .linear import main_grad_of

E4M3_MAX, E5M2_MAX = 448.0, 57344.0


def _blocks(xf, along_rows):
    """View ``xf`` [rows, cols] as [..., 32] blocks along the requested dim (zero padded)."""
    if along_rows:
        xf = xf.t()
    r, c = xf.shape
    pad = (-c) % 32
    if pad:
        xf = torch.nn.functional.pad(xf, (0, pad))
    return xf.reshape(r, -1, 32), r, c


def qdq_ref(x, along_rows=False, e5m2=False):
    """fp32 / torch statement of quantise -> dequantise (oracle and CPU path)."""
    blk, r, c = _blocks(x.float(), along_rows)
    amax = blk.abs().amax(dim=-1, keepdim=True)
    emax = 15 if e5m2 else 8
    e = torch.floor(torch.log2(amax.clamp_min(1e-38))) - emax
    e = e.clamp(-126, 127)
    scale = torch.where(amax > 0, torch.exp2(e), torch.zeros_like(amax))
    inv = torch.where(amax > 0, torch.exp2(-e), torch.zeros_like(amax))
    lim = E5M2_MAX if e5m2 else E4M3_MAX
    q = (blk * inv).clamp(-lim, lim).to(torch.float8_e5m2 if e5m2 else torch.float8_e4m3fn).float()
    out = (q * scale).reshape(r, -1)[:, :c]
    if along_rows:
        out = out.t()
    return out.contiguous().to(x.dtype)


def _kernel_ok(x):
    return x.is_cuda and native.available() and x.dtype == torch.bfloat16 and x.dim() == 2 and \
        native.lib().has("neox_mxfp8_quant")


def quantize(x, along_rows=False, e5m2=False):
    """``x`` bf16 [rows, cols] -> (fp8 bytes [rows, cols] uint8, E8M0 scales uint8 per block)."""
    assert _kernel_ok(x), "MXFP8 quantise kernel needs a CUDA bf16 matrix"
    x = x.contiguous()
    rows, cols = x.shape
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    nblk = ((rows + 31) // 32) * cols if along_rows else rows * ((cols + 31) // 32)
    s = torch.empty(nblk, dtype=torch.uint8, device=x.device)
    rc = native.lib().neox_mxfp8_quant(native.ptr(x), native.ptr(q), native.ptr(s), None, ctypes.c_longlong(rows),
                                       ctypes.c_longlong(cols), int(along_rows), int(e5m2),
                                       ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_mxfp8_quant")
    return q, s


def dequantize(q, s, along_rows=False, e5m2=False):
    rows, cols = q.shape
    out = torch.empty(rows, cols, dtype=torch.bfloat16, device=q.device)
    rc = native.lib().neox_mxfp8_dequant(native.ptr(q), native.ptr(s), native.ptr(out), ctypes.c_longlong(rows),
                                         ctypes.c_longlong(cols), int(along_rows), int(e5m2),
                                         ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_mxfp8_dequant")
    return out


def qdq(x, along_rows=False, e5m2=False):
    """Quantise to MXFP8 and back in one pass (bf16 in, bf16 out)."""
    if not _kernel_ok(x):
        return qdq_ref(x, along_rows, e5m2)
    x = x.contiguous()
    rows, cols = x.shape
    out = torch.empty_like(x)
    rc = native.lib().neox_mxfp8_quant(native.ptr(x), None, None, native.ptr(out), ctypes.c_longlong(rows),
                                       ctypes.c_longlong(cols), int(along_rows), int(e5m2),
                                       ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_mxfp8_quant")
    return out


# ------------------------------------------------------------------ hardware path (block-scaled tensor cores)
class MXTensor:
    """FP8 bytes plus E8M0 scales in the tiled layout the block-scaled MMA kernel reads (``csrc/mxfp8.cu``,
    ``sf_tiled_offset``).  ``along_rows`` says which dimension the 32-element blocks run along, i.e. which dimension
    a GEMM may contract over with this copy."""

    def __init__(self, q, sf, mnb, along_rows, e5m2):
        self.q, self.sf, self.mnb, self.along_rows, self.e5m2 = q, sf, mnb, along_rows, e5m2


def hw_ok(x):
    return _kernel_ok(x) and native.lib().has("neox_gemm_mxfp8") and x.shape[0] >= 1 and x.shape[1] % 16 == 0


def quantize_tiled(x, along_rows=False, e5m2=False) -> MXTensor:
    assert _kernel_ok(x)
    x = x.contiguous()
    rows, cols = x.shape
    mn, kdim = (cols, rows) if along_rows else (rows, cols)
    mnb = (mn + 127) // 128 + 1                      # one spare chunk: a 192-wide tile reads one chunk past its last
    kchunks = ((kdim + 31) // 32 + 3) // 4
    q = torch.empty(rows, cols, dtype=torch.uint8, device=x.device)
    sf = torch.zeros(kchunks * mnb * 512, dtype=torch.uint8, device=x.device)
    rc = native.lib().neox_mxfp8_quant_tiled(native.ptr(x), native.ptr(q), native.ptr(sf), None,
                                             ctypes.c_longlong(rows), ctypes.c_longlong(cols), int(along_rows),
                                             int(e5m2), ctypes.c_longlong(mnb), ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_mxfp8_quant_tiled")
    return MXTensor(q, sf, mnb, along_rows, e5m2)


def quantize_dual(x, e5m2=False, cols=True, rows=True):
    """One pass over ``x`` (bf16 [R, C], C % 8 == 0) producing the copy blocked along columns and / or the copy
    blocked along rows: ``(MXTensor | None, MXTensor | None)``."""
    assert _kernel_ok(x) and x.shape[1] % 8 == 0 and (cols or rows)
    x = x.contiguous()
    R, C = x.shape
    dev = x.device
    tc = tr = None
    if cols:
        mnb = (R + 127) // 128 + 1
        tc = MXTensor(torch.empty(R, C, dtype=torch.uint8, device=dev),
                      torch.zeros((((C + 31) // 32 + 3) // 4) * mnb * 512, dtype=torch.uint8, device=dev), mnb, False,
                      e5m2)
    if rows:
        mnb = (C + 127) // 128 + 1
        tr = MXTensor(torch.empty(R, C, dtype=torch.uint8, device=dev),
                      torch.zeros((((R + 31) // 32 + 3) // 4) * mnb * 512, dtype=torch.uint8, device=dev), mnb, True,
                      e5m2)
    rc = native.lib().neox_mxfp8_quant_dual(
        native.ptr(x), native.ptr(tc.q) if tc else None, native.ptr(tc.sf) if tc else None,
        ctypes.c_longlong(tc.mnb if tc else 0), native.ptr(tr.q) if tr else None, native.ptr(tr.sf) if tr else None,
        ctypes.c_longlong(tr.mnb if tr else 0), ctypes.c_longlong(R), ctypes.c_longlong(C), int(e5m2),
        ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_mxfp8_quant_dual")
    return tc, tr


def gemm_mx(a: MXTensor, b: MXTensor, out=None, out_dtype=torch.bfloat16, bias=None, add=None, act=G.ACT_NONE,
            aux=None, alpha=1.0, want_preact=False):
    """``epilogue(alpha * op(a) @ op(b))`` with the block scales applied by the tensor cores.  An operand quantised
    along its columns is used K-major (``[M, K]`` / ``[N, K]``), one quantised along its rows MN-major
    (``[K, M]`` / ``[K, N]``): either way the contraction runs along the blocked dimension."""
    a_mn, b_mn = a.along_rows, b.along_rows
    K, M = a.q.shape if a_mn else a.q.shape[::-1]
    Kb, N = b.q.shape if b_mn else b.q.shape[::-1]
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, device=a.q.device, dtype=out_dtype)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (torch.bfloat16, torch.float32)
    pre = torch.empty(M, N, device=a.q.device, dtype=torch.bfloat16) if want_preact else None
    rc = native.lib().neox_gemm_mxfp8(
        native.ptr(a.q), native.ptr(b.q), native.ptr(out), M, N, K,
        ctypes.c_longlong(a.q.stride(0)), ctypes.c_longlong(b.q.stride(0)), ctypes.c_longlong(out.stride(0)),
        int(a_mn), int(b_mn), int(a.e5m2), int(b.e5m2), native.ptr(a.sf), ctypes.c_longlong(a.mnb),
        native.ptr(b.sf), ctypes.c_longlong(b.mnb), int(out.dtype == torch.float32),
        native.ptr(bias), native.ptr(add), ctypes.c_longlong(add.stride(0) if add is not None else 0),
        int(add is not None and add.dtype == torch.float32),
        native.ptr(pre), ctypes.c_longlong(pre.stride(0) if pre is not None else 0),
        native.ptr(aux), ctypes.c_longlong(aux.stride(0) if aux is not None else 0),
        int(act), ctypes.c_float(alpha), ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_gemm_mxfp8")
    return (out, pre) if want_preact else out


_wcache: dict = {}


def _weight_mx(weight, along_rows):
    """Quantised copies of a parameter live until the optimizer step (``fp8.invalidate_weight_cache``)."""
    from . import fp8 as F8
    key = (id(weight), along_rows)
    tag = (F8._weight_epoch, weight.data_ptr(), weight._version, tuple(weight.shape))
    hit = _wcache.get(key)
    if hit is not None and hit[0] == tag:
        return hit[1]
    if len(_wcache) > 8192:
        _wcache.clear()
    if weight.shape[1] % 8 == 0:
        tc, tr = quantize_dual(weight.detach())
        _wcache[(id(weight), False)] = (tag, tc)
        _wcache[(id(weight), True)] = (tag, tr)
        return tr if along_rows else tc
    t = quantize_tiled(weight.detach(), along_rows)
    _wcache[key] = (tag, t)
    return t


class _MXLinearHwFn(torch.autograd.Function):
    """The three GEMMs of a linear layer on the block-scaled tensor cores; same quantisation points as
    ``_MXLinearFn`` (each operand blocked along the contraction dimension of the GEMM it enters)."""

    @staticmethod
    def forward(ctx, x, weight, bias, hybrid, fp8_wgrad):
        N, K = weight.shape
        x2 = x.reshape(-1, K).contiguous()
        # the copy blocked along tokens is what the weight-gradient GEMM reads: make it in the same pass and keep
        # it (fp8 + scales) instead of the bf16 activation
        keep = fp8_wgrad and torch.is_grad_enabled() and weight.requires_grad
        xc, xr = quantize_dual(x2, False, cols=True, rows=keep)
        out = gemm_mx(xc, _weight_mx(weight, False), bias=bias)
        if keep:
            ctx.save_for_backward(xr.q, xr.sf)
            ctx.xr_mnb = xr.mnb
        else:
            ctx.save_for_backward(x2)
        ctx.keep = keep
        ctx.weight = weight
        ctx.cfg = (x.shape, hybrid, fp8_wgrad, bias is not None)
        return out.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, g):
        weight = ctx.weight
        x_shape, hybrid, fp8_wgrad, has_bias = ctx.cfg
        N, K = weight.shape
        g2 = g.reshape(-1, N).contiguous()
        gx = gw = gb = None
        need_w = ctx.needs_input_grad[1]
        gc, gr = quantize_dual(g2, hybrid, cols=ctx.needs_input_grad[0], rows=need_w and fp8_wgrad) \
            if (ctx.needs_input_grad[0] or (need_w and fp8_wgrad)) else (None, None)
        if ctx.keep:
            xq, xsf = ctx.saved_tensors
            xa = MXTensor(xq, xsf, ctx.xr_mnb, True, False)
            x2 = None
        else:
            (x2,) = ctx.saved_tensors
            xa = quantize_dual(x2, False, cols=False, rows=True)[1] if (need_w and fp8_wgrad) else None
        if ctx.needs_input_grad[0]:
            gx = gemm_mx(gc, _weight_mx(weight, True)).reshape(x_shape)
        if need_w:
            mg = main_grad_of(weight)
            if fp8_wgrad:
                run = lambda **kw: gemm_mx(gr, xa, **kw)
            else:
                run = lambda **kw: G.gemm(g2, x2, a_mn=True, b_mn=True, **kw)
            if mg is not None:
                run(out=mg, add=mg)
                weight.grad_in_main = True
                from .linear import notify_grad_ready
                notify_grad_ready(weight)
            else:
                gw = run()
        if has_bias and ctx.needs_input_grad[2]:
            gb = g2.sum(0)
        return gx, gw, gb, None, None


class _MXLinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, hybrid, fp8_wgrad):
        N, K = weight.shape
        x2 = x.reshape(-1, K)
        xq = qdq(x2, along_rows=False)                   # contraction = hidden: blocks along the last dim
        wq = qdq(weight, along_rows=False)
        out = G.gemm(xq, wq, bias=bias)
        ctx.save_for_backward(x2, weight)
        ctx.cfg = (x.shape, hybrid, fp8_wgrad, bias is not None)
        return out.reshape(*x.shape[:-1], N)

    @staticmethod
    def backward(ctx, g):
        x2, weight = ctx.saved_tensors
        x_shape, hybrid, fp8_wgrad, has_bias = ctx.cfg
        N, K = weight.shape
        g2 = g.reshape(-1, N).contiguous()
        gx = gw = gb = None
        if ctx.needs_input_grad[0]:
            # dx = dy W: contraction over output features = last dim of dy, first dim of W
            gq = qdq(g2, along_rows=False, e5m2=hybrid)
            wq = qdq(weight, along_rows=True)
            gx = G.gemm(gq, wq, a_mn=False, b_mn=True).reshape(x_shape)
        if ctx.needs_input_grad[1]:
            # dW = dy^T x: contraction over tokens = first dim of both
            ga = qdq(g2, along_rows=True, e5m2=hybrid) if fp8_wgrad else g2
            xa = qdq(x2, along_rows=True) if fp8_wgrad else x2
            mg = main_grad_of(weight)
            if mg is not None:
                G.gemm(ga, xa, a_mn=True, b_mn=True, out=mg, add=mg)
                weight.grad_in_main = True
                from .linear import notify_grad_ready
                notify_grad_ready(weight)
            else:
                gw = G.gemm(ga, xa, a_mn=True, b_mn=True)
        if has_bias and ctx.needs_input_grad[2]:
            gb = g2.sum(0)
        return gx, gw, gb, None, None


HW_DEFAULT = True


def mx_linear(x, weight, bias=None, hybrid=True, fp8_wgrad=True, hardware=None):
    """``x @ weight.T + bias`` with all three GEMMs of the layer on MXFP8 operands (see module docstring).
    ``hardware``: run them on the block-scaled tensor cores (``csrc/gemm_mxfp8_sm100.cu``) instead of dequantising
    into the bf16 GEMM; ``None`` = ``NEOX_MXFP8_HW`` / the module default."""
    if hardware is None:
        import os
        hardware = os.environ.get("NEOX_MXFP8_HW", "1" if HW_DEFAULT else "0") == "1"
    N, K = weight.shape
    tokens = x.numel() // K
    if hardware and x.is_cuda and x.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and K % 16 == 0 and \
            N % 16 == 0 and tokens % 16 == 0 and native.lib().has("neox_gemm_mxfp8") and \
            (bias is None or bias.dtype == torch.bfloat16):
        return _MXLinearHwFn.apply(x, weight, bias, hybrid, fp8_wgrad)
    return _MXLinearFn.apply(x, weight, bias, hybrid, fp8_wgrad)
