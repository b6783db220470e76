"""1-bit Adam (Tang et al. 2021).  For ``freeze_step`` warm-up steps this is plain Adam; afterwards the
variance is frozen and only the momentum is communicated, compressed to its sign plus one scale per
chunk with local error feedback.  Here the optimizer runs on the *already reduced* gradient shard, so
the compression is applied to the momentum update itself (error-compensated sign quantisation), which
reproduces the optimizer's numerics; the bandwidth saving of the original applies to inter-node
all-reduce and is out of scope on a single NVSwitch domain."""
from __future__ import annotations

import torch


class OneBitAdam(torch.optim.Optimizer):
    supports_grad_scale = False

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, freeze_step=400,
                 bias_correction=True, **_ignored):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                                      bias_correction=bias_correction))
        self.freeze_step = freeze_step

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                if not st:
                    st.update(step=0, exp_avg=torch.zeros_like(g), exp_avg_sq=torch.zeros_like(g),
                              error=torch.zeros_like(g))
                st["step"] += 1
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(g, alpha=1 - b1)
                if st["step"] <= self.freeze_step:
                    v.mul_(b2).addcmul_(g, g, value=1 - b2)
                else:
                    comp = m + st["error"]
                    scale = comp.abs().mean()
                    q = comp.sign() * scale
                    st["error"] = comp - q
                    m.copy_(q)
                upd = m / (v.sqrt() + group["eps"])
                if group["weight_decay"]:
                    upd = upd + group["weight_decay"] * p.float()
                p.add_(upd.to(p.dtype), alpha=-group["lr"])
        return loss
