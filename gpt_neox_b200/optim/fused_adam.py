"""Adam / AdamW whose update is one fused kernel over a flat fp32 shard.

For every parameter (normally the single flat master shard of a bucket) one launch of
``neox_adam_step`` reads the fp32 gradient, multiplies it by ``grad_scale`` (un-scaling and clipping
folded in), updates ``m``, ``v`` and the fp32 master weight and, when the parameter carries a
``model_out`` tensor, also writes the bf16/fp16 copy consumed by the forward pass -- replacing apex's
``multi_tensor_adam`` plus the separate fp32->bf16 copy of the reference stack
(``megatron/training.py:1159-1173``).  On CPU the same update is evaluated with torch ops.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import native
from ..ops.functional import _DT


class FusedAdam(torch.optim.Optimizer):
    supports_grad_scale = True
    writes_model_out = True

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, adam_w_mode=True,
                 bias_correction=True, amsgrad=False, **_ignored):
        if amsgrad:
            raise RuntimeError("FusedAdam does not support the AMSGrad variant.")
        defaults = dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, bias_correction=bias_correction,
                        grad_scale=1.0)
        super().__init__(params, defaults)
        self.adam_w_mode = bool(adam_w_mode)

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            group["step"] = group.get("step", 0) + 1
            t = group["step"]
            if group["bias_correction"]:
                bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
            else:
                bc1 = bc2 = 1.0
            gs = float(group.get("grad_scale", 1.0))
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p, dtype=torch.float32)
                m, v, g = st["exp_avg"], st["exp_avg_sq"], p.grad
                out = getattr(p, "model_out", None)
                if p.is_cuda and native.available() and p.dtype == torch.float32 and g.dtype == torch.float32:
                    rc = native.lib().neox_adam_step(
                        native.ptr(p), native.ptr(m), native.ptr(v), native.ptr(g), native.ptr(out),
                        _DT[out.dtype] if out is not None else 1, ctypes.c_longlong(p.numel()),
                        ctypes.c_float(group["lr"]), ctypes.c_float(b1), ctypes.c_float(b2),
                        ctypes.c_float(group["eps"]), ctypes.c_float(group["weight_decay"]), ctypes.c_float(bc1),
                        ctypes.c_float(bc2), ctypes.c_float(gs), int(self.adam_w_mode),
                        ctypes.c_void_p(native.stream_ptr()))
                    native.check(rc, "neox_adam_step")
                else:
                    gf = g.float() * gs
                    if not self.adam_w_mode and group["weight_decay"] != 0:
                        gf = gf + group["weight_decay"] * p
                    m.mul_(b1).add_(gf, alpha=1 - b1)
                    v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
                    denom = (v / bc2).sqrt_().add_(group["eps"])
                    upd = (m / bc1) / denom
                    if self.adam_w_mode and group["weight_decay"] != 0:
                        upd = upd + group["weight_decay"] * p
                    p.add_(upd, alpha=-group["lr"])
                    if out is not None:
                        out.copy_(p)
        return loss
