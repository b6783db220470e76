"""16-bit (bf16 / fp16) GEMM front-end for the tcgen05 kernels in ``csrc/gemm_sm100.cu`` and ``csrc/gemm_2cta_sm100.cu``.

``gemm(a, b, ...)`` computes ``epilogue(alpha * op(a) @ op(b))`` where each operand is given as a
2-D tensor and a flag telling whether it is stored "K-major" (contraction index contiguous) or
"MN-major".  The three GEMMs of a linear layer map onto it without any transposition copy:

=========  =======================  ==================  ==================
pass       math                     A (stored)          B (stored)
=========  =======================  ==================  ==================
forward    Y[M,N] = X W^T           X[M,K]  K-major     W[N,K]  K-major
dgrad      dX[M,K] = dY W           dY[M,N] K-major     W[N,K]  MN-major
wgrad      dW[N,K] = dY^T X         dY[M,N] MN-major    X[M,K]  MN-major
=========  =======================  ==================  ==================

On CPU (no device) the same function evaluates the identical math with torch ops in fp32, which is
the oracle the GPU tests compare against.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import flop_count, native

ACT_NONE, ACT_GELU, ACT_DGELU = 0, 1, 2


def gelu_tanh_ref(x):
    return F.gelu(x, approximate="tanh")


def dgelu_tanh_ref(x):
    k0, k1 = 0.7978845608028654, 0.044715
    t = torch.tanh(k0 * x * (1 + k1 * x * x))
    return 0.5 * x * ((1 - t * t) * (k0 + 3 * k0 * k1 * x * x)) + 0.5 * (1 + t)


def gemm_ref(a, b, a_mn=False, b_mn=False, out_dtype=torch.bfloat16, bias=None, add=None, act=ACT_NONE, aux=None,
             alpha=1.0, want_preact=False):
    """fp32 eager statement of the kernel's math (oracle and CPU path)."""
    A = a.float().t() if a_mn else a.float()          # [M, K]
    B = b.float() if b_mn else b.float().t()          # [K, N]
    v = alpha * (A @ B)
    if bias is not None:
        v = v + bias.float()
    pre = v.to(a.dtype if a.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16) if want_preact else None
    if act == ACT_GELU:
        v = gelu_tanh_ref(v)
    elif act == ACT_DGELU:
        v = v * dgelu_tanh_ref(aux.float())
    if add is not None:
        v = v + add.float()
    v = v.to(out_dtype)
    return (v, pre) if want_preact else v


_PAIR = None


def use_pair_kernel(M, N, K):
    """The CTA-pair kernel (``csrc/gemm_2cta_sm100.cu``, 256 x 256 tiles on two SMs) pays off once the problem
    fills the machine with such tiles; small problems keep the one-CTA kernel.  ``NEOX_GEMM_2CTA=0/1`` forces it."""
    global _PAIR
    if _PAIR is None:
        import os
        _PAIR = os.environ.get("NEOX_GEMM_2CTA", "auto")
    if _PAIR == "0":
        return False
    if _PAIR == "1":
        return True
    return PAIR_DEFAULT and ((M + 255) // 256) * ((N + 255) // 256) >= 74 and K >= 256


PAIR_DEFAULT = True


def gemm_rowmap(a, b, row_ptrs, b_mn=False, bias=None):
    """``a @ op(b) + bias`` whose output row r is stored (bf16) at device address ``row_ptrs[r]`` (int64 tensor of
    M addresses, 16-byte aligned, possibly in other GPUs' peer-mapped memory) instead of into one matrix."""
    assert a.is_cuda and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16 and row_ptrs.dtype == torch.int64
    M, K = a.shape
    N = b.shape[1] if b_mn else b.shape[0]
    assert row_ptrs.numel() == M and N % 8 == 0
    if M == 0:
        return
    rc = native.lib().neox_gemm_bf16_rowmap(
        native.ptr(a), native.ptr(b), None, M, N, K, ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)),
        ctypes.c_longlong(N), 0, int(b_mn), 0, native.ptr(bias), None, ctypes.c_longlong(0), 0, None,
        ctypes.c_longlong(0), None, ctypes.c_longlong(0), ACT_NONE, ctypes.c_float(1.0), native.ptr(row_ptrs),
        ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_gemm_bf16_rowmap")


def gemm(a, b, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16, bias=None, add=None, act=ACT_NONE,
         aux=None, alpha=1.0, want_preact=False):
    """See module docstring.  ``add`` may alias ``out`` (in-place accumulate, e.g. wgrad into main_grad)."""
    if flop_count.ACTIVE[0] is not None:
        flop_count.gemm(a.shape[0], b.shape[1] if b_mn else b.shape[0], a.shape[1]) if not a_mn else \
            flop_count.gemm(a.shape[1], b.shape[1] if b_mn else b.shape[0], a.shape[0])
    if not a.is_cuda:
        r = gemm_ref(a, b, a_mn, b_mn, out_dtype if out is None else out.dtype, bias, add, act, aux, alpha, want_preact)
        if out is not None:
            if want_preact:
                out.copy_(r[0]); return out, r[1]
            out.copy_(r); return out
        return r
    dt = a.dtype
    assert dt in (torch.bfloat16, torch.float16) and b.dtype == dt, "tcgen05 GEMM takes two bf16 or two fp16 operands"
    if out is None and out_dtype == torch.bfloat16:
        out_dtype = dt                      # the default output type is the operand type
    assert a.dim() == 2 and b.dim() == 2 and a.stride(1) == 1 and b.stride(1) == 1
    if a_mn:
        K, M = a.shape
    else:
        M, K = a.shape
    if b_mn:
        Kb, N = b.shape
    else:
        N, Kb = b.shape
    assert K == Kb, f"contraction mismatch {K} vs {Kb}"
    if out is None:
        out = torch.empty(M, N, device=a.device, dtype=out_dtype)
    assert out.shape == (M, N) and out.stride(1) == 1 and out.dtype in (dt, torch.float32)
    pre = torch.empty(M, N, device=a.device, dtype=dt) if want_preact else None
    if add is not None:
        assert add.shape == (M, N) and add.stride(1) == 1 and add.dtype in (dt, torch.float32)
    if bias is not None:
        assert bias.dtype == dt and bias.numel() == N and bias.is_contiguous()
    if act == ACT_DGELU:
        assert aux is not None and aux.shape == (M, N) and aux.dtype == dt and aux.stride(1) == 1
    L = native.lib()
    h16 = int(dt == torch.float16)
    pair = use_pair_kernel(M, N, K)
    tail = (h16, ctypes.c_void_p(native.stream_ptr())) if pair else (None, h16, ctypes.c_void_p(native.stream_ptr()))
    fn = L.neox_gemm_16_2cta if pair else L.neox_gemm_16
    rc = fn(
        native.ptr(a), native.ptr(b), native.ptr(out), M, N, K,
        ctypes.c_longlong(a.stride(0)), ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0)),
        int(a_mn), int(b_mn), int(out.dtype == torch.float32),
        native.ptr(bias), native.ptr(add), ctypes.c_longlong(add.stride(0) if add is not None else 0),
        int(add is not None and add.dtype == torch.float32),
        native.ptr(pre), ctypes.c_longlong(pre.stride(0) if pre is not None else 0),
        native.ptr(aux), ctypes.c_longlong(aux.stride(0) if aux is not None else 0),
        int(act), ctypes.c_float(alpha), *tail)
    native.check(rc, "neox_gemm_16")
    return (out, pre) if want_preact else out
