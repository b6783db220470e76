"""MADGRAD with decoupled weight decay (Defazio & Jelassi 2021): a momentumised dual-averaging
AdaGrad.  With ``lamb = lr * sqrt(k+1)``: ``s += lamb*g``, ``v += lamb*g^2``,
``z = x0 - s / (cbrt(v) + eps)``, ``x <- (1-ck)*x + ck*z`` with ``ck = 1 - momentum``.
Element-wise, so it runs on the flat fp32 shard.  Reference: ``megatron/optimizers.py:242-415``."""
from __future__ import annotations

import math

import torch


class madgrad_wd(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-2, momentum: float = 0.9, weight_decay: float = 0, eps: float = 1e-6,
                 **_ignored):
        if momentum < 0 or momentum >= 1:
            raise ValueError(f"Momentum {momentum} must be in the range [0,1]")
        if lr <= 0:
            raise ValueError(f"Learning rate {lr} must be positive")
        if weight_decay < 0:
            raise ValueError(f"Weight decay {weight_decay} must be non-negative")
        if eps < 0:
            raise ValueError("Eps must be non-negative")
        super().__init__(params, dict(lr=lr, eps=eps, momentum=momentum, weight_decay=weight_decay, k=0))

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            eps, lr, wd, mom = group["eps"], group["lr"] + group["eps"], group["weight_decay"], group["momentum"]
            k = group.get("k", 0)
            ck = 1 - mom
            lamb = lr * math.sqrt(k + 1)
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                if not st:
                    st["grad_sum_sq"] = torch.zeros_like(p, dtype=torch.float32)
                    st["s"] = torch.zeros_like(p, dtype=torch.float32)
                    if mom != 0:
                        st["x0"] = p.detach().clone().float()
                if wd:
                    p.mul_(1 - group["lr"] * wd)
                v, s = st["grad_sum_sq"], st["s"]
                if mom == 0:
                    rms = v.pow(1 / 3).add_(eps)
                    x0 = p.float().addcdiv(s, rms, value=1)
                else:
                    x0 = st["x0"]
                v.addcmul_(g, g, value=lamb)
                rms = v.pow(1 / 3).add_(eps)
                s.add_(g, alpha=lamb)
                if mom == 0:
                    p.copy_(x0.addcdiv(s, rms, value=-1))
                else:
                    z = x0.addcdiv(s, rms, value=-1)
                    p.mul_(1 - ck).add_(z.to(p.dtype), alpha=ck)
            group["k"] = k + 1
        return loss
