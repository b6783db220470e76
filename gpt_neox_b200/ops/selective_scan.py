"""Mamba selective scan (S6) and causal depth-wise conv1d.

    delta = softplus(dt + dt_bias);  h_t = exp(delta_t A) * h_{t-1} + delta_t B_t u_t;  y_t = C_t . h_t + D u_t
    out = y * silu(z)

Layouts are channel-last -- u, dt, z ``[b, l, d]``, B, C ``[b, l, n]`` -- so consecutive threads of the CUDA
kernel (``csrc/selective_scan.cu``, one thread per channel, state in registers, checkpointed every 32 steps for
the backward recomputation) touch consecutive addresses and no ``b d l`` transposes are needed.
``selective_scan_ref`` states the same recurrence in PyTorch (CPU path and oracle).
Reference: mamba_ssm ``selective_scan_fn`` / ``causal_conv1d_fn`` as called from ``megatron/model/mamba/mamba.py:207-300``.
"""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import native


def selective_scan_ref(u, dt, A, B, C, D=None, z=None, dt_bias=None, dt_softplus=True):
    b, l, d = u.shape
    n = A.shape[1]
    uf, dtf = u.float(), dt.float()
    if dt_bias is not None:
        dtf = dtf + dt_bias.float()
    if dt_softplus:
        dtf = F.softplus(dtf)
    Af, Bf, Cf = A.float(), B.float(), C.float()
    h = torch.zeros(b, d, n, dtype=torch.float32, device=u.device)
    ys = []
    for t in range(l):
        dA = torch.exp(dtf[:, t, :, None] * Af[None])                    # [b, d, n]
        dBu = dtf[:, t, :, None] * Bf[:, t, None, :] * uf[:, t, :, None]
        h = dA * h + dBu
        ys.append(torch.einsum("bdn,bn->bd", h, Cf[:, t]))
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + uf * D.float()
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(u.dtype)


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, dt, A, B, C, D, z, dt_bias):
        b, l, d = u.shape
        n = A.shape[1]
        u, dt, z = u.contiguous(), dt.contiguous(), z.contiguous()
        Bc, Cc = B.float().contiguous(), C.float().contiguous()
        Af, Df, bias = A.float().contiguous(), D.float().contiguous(), dt_bias.float().contiguous()
        nchk = (l + 31) // 32
        y = torch.empty_like(u)
        ckpt = torch.empty(b, nchk, d, n, dtype=torch.float32, device=u.device)
        rc = native.lib().neox_selective_scan_fwd(native.ptr(u), native.ptr(dt), native.ptr(Af), native.ptr(Bc),
                                                  native.ptr(Cc), native.ptr(Df), native.ptr(z), native.ptr(bias),
                                                  native.ptr(y), native.ptr(ckpt), b, l, d, n,
                                                  ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_selective_scan_fwd")
        ctx.save_for_backward(u, dt, Af, Bc, Cc, Df, z, bias, ckpt)
        ctx.dtypes = (A.dtype, B.dtype, C.dtype, D.dtype, dt_bias.dtype)
        return y

    @staticmethod
    def backward(ctx, gy):
        u, dt, Af, Bc, Cc, Df, z, bias, ckpt = ctx.saved_tensors
        b, l, d = u.shape
        n = Af.shape[1]
        gy = gy.contiguous()
        du, ddt, dz = torch.empty_like(u), torch.empty_like(dt), torch.empty_like(z)
        dA = torch.zeros(d, n, dtype=torch.float32, device=u.device)
        dB = torch.zeros(b, l, n, dtype=torch.float32, device=u.device)
        dC = torch.zeros(b, l, n, dtype=torch.float32, device=u.device)
        dD = torch.zeros(d, dtype=torch.float32, device=u.device)
        dbias = torch.zeros(d, dtype=torch.float32, device=u.device)
        rc = native.lib().neox_selective_scan_bwd(native.ptr(u), native.ptr(dt), native.ptr(Af), native.ptr(Bc),
                                                  native.ptr(Cc), native.ptr(Df), native.ptr(z), native.ptr(bias),
                                                  native.ptr(ckpt), native.ptr(gy), native.ptr(du), native.ptr(ddt),
                                                  native.ptr(dz), native.ptr(dA), native.ptr(dB), native.ptr(dC),
                                                  native.ptr(dD), native.ptr(dbias), b, l, d, n,
                                                  ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_selective_scan_bwd")
        ta, tb, tc, td, tbias = ctx.dtypes
        return du, ddt, dA.to(ta), dB.to(tb), dC.to(tc), dD.to(td), dz, dbias.to(tbias)


def have_scan_kernel():
    return native.available() and native.lib().has("neox_selective_scan_fwd")


def selective_scan(u, dt, A, B, C, D, z, dt_bias):
    """All of D, z, dt_bias are required on the kernel path (the Mamba block always has them)."""
    if u.is_cuda and u.dtype == torch.bfloat16 and A.shape[1] == 16 and have_scan_kernel():
        return _Scan.apply(u, dt, A, B, C, D, z, dt_bias)
    return selective_scan_ref(u, dt, A, B, C, D, z, dt_bias, True)


def causal_conv1d(x, weight, bias, activation="silu"):
    """Depth-wise causal conv over time for channel-last ``x`` ``[b, l, d]``; ``weight`` ``[d, w]``."""
    w = weight.shape[1]
    y = F.conv1d(x.transpose(1, 2), weight.unsqueeze(1), bias, padding=w - 1, groups=weight.shape[0])[..., : x.shape[1]]
    y = y.transpose(1, 2)
    return F.silu(y) if activation == "silu" else y
