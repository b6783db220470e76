"""Lion (EvoLved Sign Momentum; Chen et al. 2023): ``update = sign(b1*m + (1-b1)*g)``,
``p <- p*(1 - lr*wd) - lr*update``, ``m <- b2*m + (1-b2)*g``.  Element-wise, so it runs on the flat
fp32 shard; on CUDA the step is one fused kernel (``neox_lion_step``) that also writes the
bf16 copy.  Reference: ``megatron/optimizers.py:418-497`` and DeepSpeed's FusedLion."""
from __future__ import annotations

import ctypes

import torch

from ..ops import native
from ..ops.functional import _DT


class Lion(torch.optim.Optimizer):
    supports_grad_scale = True
    writes_model_out = True

    def __init__(self, params, lr: float = 1e-4, betas=(0.9, 0.99), weight_decay: float = 0.0, **_ignored):
        if lr <= 0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not all(0.0 <= b <= 1.0 for b in betas):
            raise ValueError(f"Invalid beta: {betas}")
        super().__init__(params, dict(lr=lr, betas=tuple(betas), weight_decay=weight_decay, grad_scale=1.0))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            gs = float(group.get("grad_scale", 1.0))
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["exp_avg"] = torch.zeros_like(p, dtype=torch.float32)
                m, g = st["exp_avg"], p.grad
                out = getattr(p, "model_out", None)
                if p.is_cuda and native.available() and p.dtype == torch.float32 and g.dtype == torch.float32:
                    rc = native.lib().neox_lion_step(native.ptr(p), native.ptr(m), native.ptr(g), native.ptr(out),
                                                     _DT[out.dtype] if out is not None else 1,
                                                     ctypes.c_longlong(p.numel()), ctypes.c_float(group["lr"]),
                                                     ctypes.c_float(b1), ctypes.c_float(b2),
                                                     ctypes.c_float(group["weight_decay"]), ctypes.c_float(gs),
                                                     ctypes.c_void_p(native.stream_ptr()))
                    native.check(rc, "neox_lion_step")
                else:
                    gf = g.float() * gs
                    p.mul_(1 - group["lr"] * group["weight_decay"])
                    upd = (m * b1 + gf * (1 - b1)).sign_()
                    p.add_(upd, alpha=-group["lr"])
                    m.mul_(b2).add_(gf, alpha=1 - b2)
                    if out is not None:
                        out.copy_(p)
        return loss
