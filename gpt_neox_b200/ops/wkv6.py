"""RWKV-6 wkv operator: CUDA kernels (``csrc/wkv6.cu``) with a PyTorch statement of the same recurrence as the
CPU path and test oracle.  ``wkv6(r, k, v, w, u)`` takes ``[B, T, C]`` tensors (C = H * N), the per-channel decay
logits ``w`` (the decay is ``exp(-exp(w))``) and the bonus ``u`` ``[H, N]``."""
from __future__ import annotations

import ctypes

import torch

from . import native


def wkv6_ref(r, k, v, w, u):
    B, T, C = r.shape
    H, N = u.shape
    rf, kf, vf = (t.float().view(B, T, H, N) for t in (r, k, v))
    d = torch.exp(-torch.exp(w.float())).view(B, T, H, N)
    uf = u.float()
    S = torch.zeros(B, H, N, N, dtype=torch.float32, device=r.device)      # [j, i]
    ys = []
    for t in range(T):
        kv = kf[:, t, :, :, None] * vf[:, t, :, None, :]                   # [B, H, j, i]
        y = torch.einsum("bhj,bhji->bhi", rf[:, t], uf[None, :, :, None] * kv + S)
        ys.append(y)
        S = S * d[:, t, :, :, None] + kv
    return torch.stack(ys, dim=1).reshape(B, T, C).to(r.dtype)


class _WKV6(torch.autograd.Function):
    @staticmethod
    def forward(ctx, r, k, v, w, u):
        B, T, C = r.shape
        H = u.shape[0]
        r, k, v = r.contiguous(), k.contiguous(), v.contiguous()
        ew = (-torch.exp(w.float())).contiguous()
        ub = u.to(torch.bfloat16).contiguous()
        y = torch.empty_like(r)
        rc = native.lib().neox_wkv6_fwd(B, T, C, H, native.ptr(r), native.ptr(k), native.ptr(v), native.ptr(ew),
                                        native.ptr(ub), native.ptr(y), ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_wkv6_fwd")
        ctx.save_for_backward(r, k, v, ew, ub)
        ctx.u_dtype = u.dtype
        return y

    @staticmethod
    def backward(ctx, gy):
        r, k, v, ew, ub = ctx.saved_tensors
        B, T, C = r.shape
        H, N = ub.shape
        gy = gy.contiguous()
        gr, gk, gv = torch.empty_like(r), torch.empty_like(r), torch.empty_like(r)
        grS = torch.empty(B, T, C, dtype=torch.float32, device=r.device)
        gkG = torch.empty(B, T, C, dtype=torch.float32, device=r.device)
        gu_part = torch.empty(B, H, N, dtype=torch.float32, device=r.device)
        rc = native.lib().neox_wkv6_bwd(B, T, C, H, native.ptr(r), native.ptr(k), native.ptr(v), native.ptr(ew),
                                        native.ptr(ub), native.ptr(gy), native.ptr(gr), native.ptr(gk),
                                        native.ptr(gv), native.ptr(grS), native.ptr(gkG), native.ptr(gu_part),
                                        ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_wkv6_bwd")
        # d_t * dL/dd_t = sum_{s>t} r_s grS_s - sum_{s>=t} k_s gkG_s   (reverse cumulative sums over time)
        a = r.float() * grS
        b = k.float() * gkG
        ra = torch.flip(torch.cumsum(torch.flip(a, [1]), 1), [1]) - a
        rb = torch.flip(torch.cumsum(torch.flip(b, [1]), 1), [1])
        gw = ((ra - rb) * ew).to(r.dtype)
        return gr, gk, gv, gw, gu_part.sum(0).to(ctx.u_dtype)


def wkv6(r, k, v, w, u):
    if r.is_cuda and native.available() and r.dtype == torch.bfloat16 and (r.shape[-1] // u.shape[0]) in (32, 64, 128):
        return _WKV6.apply(r, k, v, w.to(torch.bfloat16) if w.dtype != torch.bfloat16 else w, u)
    return wkv6_ref(r, k, v, w, u)
