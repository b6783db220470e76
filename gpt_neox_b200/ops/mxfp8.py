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
            mg = getattr(weight, "main_grad", None)
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


def mx_linear(x, weight, bias=None, hybrid=True, fp8_wgrad=True):
    """``x @ weight.T + bias`` with all three GEMMs of the layer on MXFP8 operands (see module docstring)."""
    return _MXLinearFn.apply(x, weight, bias, hybrid, fp8_wgrad)
