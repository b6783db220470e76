"""1-bit Adam (Tang et al. 2021; the reference reaches DeepSpeed's ``OnebitAdam`` through ``optimizer.type:
OneBitAdam``, ``megatron/training.py:1013-1024``).

Two phases.  For ``freeze_step`` warm-up steps this is plain Adam on gradients that the engine has already averaged
over the data-parallel group.  Afterwards the second moment is frozen and the *gradients are no longer reduced at
all*: every rank folds its local gradient into its momentum, and the momentum is averaged over the data-parallel group
by ``compressed_allreduce`` -- one sign bit per element plus one fp32 scale per rank and chunk, with error feedback on
both the sending ("worker") and the reducing ("server") side, so the quantisation error of one step is re-injected
into the next instead of being lost.  Per step and rank that moves ``n/8 + n/(8 world)`` bytes instead of the ``8 n``
bytes of an fp32 ring all-reduce.

``compression_active`` tells the mixed-precision optimizer wrapper (``engine/flat_optimizer.py``) to skip its own
gradient reduction; compression needs every rank to hold the whole parameter (ZeRO stage 0), as DeepSpeed's does.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist


def pack_signs(x: torch.Tensor) -> torch.Tensor:
    """One bit per element (1 = non-negative), eight elements per byte; ``x.numel()`` must be a multiple of 8."""
    bits = (x >= 0).to(torch.uint8).view(-1, 8)
    weights = torch.tensor([1, 2, 4, 8, 16, 32, 64, 128], dtype=torch.uint8, device=x.device)
    return (bits * weights).sum(dim=1, dtype=torch.uint8)


def unpack_signs(packed: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Inverse of ``pack_signs``: a tensor of +1 / -1."""
    shifts = torch.arange(8, dtype=torch.uint8, device=packed.device)
    bits = (packed.view(-1, 1) >> shifts) & 1
    return bits.to(dtype).mul_(2).sub_(1).view(-1)


def _compress(buf, error):
    """``buf + error`` as (packed signs, scale) with the new quantisation error written back to ``error``."""
    buf = buf + error
    scale = buf.norm() / math.sqrt(buf.numel())
    packed = pack_signs(buf)
    error.copy_(buf - scale * unpack_signs(packed, buf.dtype))
    return packed, scale


def compressed_allreduce(buf, worker_error, server_error, group=None):
    """Average ``buf`` (fp32, numel a multiple of ``8 * world``) over ``group`` exchanging sign bits and scales only.

    worker: compress ``buf + worker_error`` -> every rank receives the chunk it serves from every rank;
    server: average the de-quantised chunks, compress ``avg + server_error`` -> all-gather signs and scales.
    ``worker_error`` has the size of ``buf``, ``server_error`` the size of one chunk.  Returns the averaged tensor
    (the same on every rank)."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    n = buf.numel()
    if world == 1:
        packed, scale = _compress(buf, worker_error)
        return scale * unpack_signs(packed, buf.dtype)
    assert n % (8 * world) == 0, "pad the buffer to a multiple of 8 * world elements"
    chunk = n // world
    rank = dist.get_rank(group)
    packed, scale = _compress(buf, worker_error)
    # ---- signs of chunk r go to rank r; scales go to everybody
    scales = torch.empty(world, dtype=buf.dtype, device=buf.device)
    dist.all_gather_into_tensor(scales, scale.reshape(1), group=group)
    recv = torch.empty(world, chunk // 8, dtype=torch.uint8, device=buf.device)
    if dist.get_backend(group) == "nccl":
        dist.all_to_all_single(recv.view(-1), packed, group=group)
    else:
        everything = torch.empty(world, n // 8, dtype=torch.uint8, device=buf.device)
        dist.all_gather_into_tensor(everything.view(-1), packed, group=group)
        recv.copy_(everything[:, rank * (chunk // 8):(rank + 1) * (chunk // 8)])
    # ---- server side: average my chunk, compress again
    avg = (unpack_signs(recv.view(-1), buf.dtype).view(world, chunk) * scales.view(world, 1)).sum(0) / world
    s_packed, s_scale = _compress(avg, server_error)
    all_packed = torch.empty(world, chunk // 8, dtype=torch.uint8, device=buf.device)
    dist.all_gather_into_tensor(all_packed.view(-1), s_packed, group=group)
    s_scales = torch.empty(world, dtype=buf.dtype, device=buf.device)
    dist.all_gather_into_tensor(s_scales, s_scale.reshape(1), group=group)
    return (unpack_signs(all_packed.view(-1), buf.dtype).view(world, chunk) * s_scales.view(world, 1)).view(-1)


class OneBitAdam(torch.optim.Optimizer):
    supports_grad_scale = False
    rank_local_state = True         # the error-feedback buffers differ per rank: every rank checkpoints its own state

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.0, freeze_step=400,
                 bias_correction=True, comm_group=None, **_ignored):
        super().__init__(params, dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay,
                                      bias_correction=bias_correction))
        self.freeze_step = int(freeze_step)
        self.comm_group = comm_group
        self.steps_done = 0

    @property
    def compression_active(self) -> bool:
        """True once the warm-up is over: the NEXT step consumes local (unreduced) gradients and communicates the
        momentum in compressed form."""
        return self.steps_done >= self.freeze_step

    def _world(self):
        return dist.get_world_size(self.comm_group) if dist.is_available() and dist.is_initialized() else 1

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        compressed = self.compression_active
        world = self._world()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad.float()
                st = self.state[p]
                if not st:
                    st.update(step=0, exp_avg=torch.zeros_like(g), exp_avg_sq=torch.zeros_like(g))
                st["step"] += 1
                m, v = st["exp_avg"], st["exp_avg_sq"]
                m.mul_(b1).add_(g, alpha=1 - b1)
                if not compressed:
                    v.mul_(b2).addcmul_(g, g, value=1 - b2)
                else:
                    n = m.numel()
                    padded = (n + 8 * world - 1) // (8 * world) * (8 * world)
                    if "worker_error" not in st:
                        st["worker_error"] = torch.zeros(padded, dtype=m.dtype, device=m.device)
                        st["server_error"] = torch.zeros(padded // world, dtype=m.dtype, device=m.device)
                    flat = m.reshape(-1)
                    if padded != n:
                        flat = torch.cat([flat, flat.new_zeros(padded - n)])
                    out = compressed_allreduce(flat, st["worker_error"], st["server_error"], self.comm_group)
                    m.copy_(out[:n].view_as(m))
                upd = m / (v.sqrt() + group["eps"])
                if group["weight_decay"]:
                    upd = upd + group["weight_decay"] * p.float()
                p.add_(upd.to(p.dtype), alpha=-group["lr"])
        self.steps_done += 1
        return loss

    def state_dict(self):
        sd = super().state_dict()
        sd["steps_done"] = self.steps_done
        return sd

    def load_state_dict(self, sd):
        sd = dict(sd)
        self.steps_done = int(sd.pop("steps_done", 0))
        super().load_state_dict(sd)
