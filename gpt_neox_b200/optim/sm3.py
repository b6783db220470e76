"""SM3 (Anil et al. 2019, "Memory-Efficient Adaptive Optimization"): Adagrad-like second moments kept
as one accumulator per tensor *axis* (cover sets = rows, columns, ...), so memory is sub-linear in
the parameter count.  Reference implementation: ``megatron/optimizers.py:20-215``."""
from __future__ import annotations

import torch


class SM3(torch.optim.Optimizer):
    def __init__(self, params, lr=0.1, momentum=0.0, beta=0.0, eps=1e-30, **_ignored):
        if not 0.0 <= lr:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= momentum < 1.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        if not 0.0 <= beta < 1.0:
            raise ValueError(f"Invalid beta: {beta}")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid eps: {eps}")
        super().__init__(params, dict(lr=lr, momentum=momentum, beta=beta, eps=eps))

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            mom, beta, eps, lr = group["momentum"], group["beta"], group["eps"], group["lr"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                if g.is_sparse:
                    raise RuntimeError("SM3 here does not support sparse gradients")
                st = self.state[p]
                rank = g.dim()
                if not st:
                    st["step"] = 0
                    st["momentum_buffer"] = torch.zeros_like(g) if mom > 0 else None
                    if rank == 0:
                        st["accumulator_0"] = torch.zeros_like(g)
                    for i in range(rank):
                        shape = [1] * rank
                        shape[i] = g.shape[i]
                        st[f"accumulator_{i}"] = torch.zeros(shape, dtype=g.dtype, device=g.device)
                # nu = min over axes of the per-axis accumulators (broadcast)
                nu = st["accumulator_0"]
                for i in range(1, rank):
                    nu = torch.min(nu, st[f"accumulator_{i}"])
                nu = nu.expand_as(g) if rank > 0 else nu
                if beta > 0:
                    nu = nu * beta
                    upd = nu + (1 - beta) * g * g
                else:
                    upd = nu + g * g
                # push the new maxima back to every axis accumulator
                if rank == 0:
                    st["accumulator_0"] = upd.clone()
                for i in range(rank):
                    acc = upd
                    for j in range(rank):
                        if j != i:
                            acc = acc.max(dim=j, keepdim=True).values
                    st[f"accumulator_{i}"] = torch.max(st[f"accumulator_{i}"], acc) if beta == 0 else acc
                step = g / (upd.sqrt() + eps)
                if mom > 0:
                    buf = st["momentum_buffer"]
                    buf.mul_(mom).add_(step, alpha=1 - mom)
                    step = buf
                p.add_(step.to(p.dtype), alpha=-lr)
                st["step"] += 1
        return loss
