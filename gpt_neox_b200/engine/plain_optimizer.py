"""Thin adapter giving a shape-aware ``torch.optim.Optimizer`` (SM3) the interface the engine expects
from ``FlatMixedPrecisionOptimizer``: data-parallel gradient all-reduce, global-norm clipping, step."""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..parallel import mpu
from .loss_scaler import StaticLossScaler


class PlainOptimizer:
    zero_stage = 0

    def __init__(self, optimizer, clip_grad=0.0):
        self.optimizer = optimizer
        self.param_groups = optimizer.param_groups
        self.clip_grad = float(clip_grad or 0.0)
        self.loss_scaler = StaticLossScaler(1.0)
        self.overflow = False
        self.skipped_steps = 0
        self._global_grad_norm = 0.0
        self.buckets = []

    @property
    def cur_scale(self):
        return 1.0

    def scale_loss(self, loss):
        return loss

    def zero_grad(self, set_to_none=True):
        self.optimizer.zero_grad(set_to_none=True)

    def _params(self):
        return [p for g in self.param_groups for p in g["params"] if p.grad is not None]

    def step(self, grad_divisor=1.0):
        params = self._params()
        dp = mpu.get_data_parallel_world_size()
        for p in params:
            if dp > 1:
                dist.all_reduce(p.grad, group=mpu.get_data_parallel_group())
            p.grad.div_(grad_divisor)
        tp_rank = mpu.get_model_parallel_rank()
        sq = sum((p.grad.float().pow(2).sum() for p in params
                  if getattr(p, "model_parallel", False) or tp_rank == 0), torch.zeros(()))
        if mpu.get_model_parallel_world_size() > 1:
            dist.all_reduce(sq, group=mpu.get_model_parallel_group())
        norm = float(sq.sqrt())
        self._global_grad_norm = norm
        if not math.isfinite(norm):
            self.overflow = True
            self.skipped_steps += 1
            self.zero_grad()
            return False
        self.overflow = False
        if self.clip_grad > 0 and norm > self.clip_grad:
            for p in params:
                p.grad.mul_(self.clip_grad / norm)
        self.optimizer.step()
        self.zero_grad()
        return True

    def state_dict(self):
        return {"optimizer_state_dict": self.optimizer.state_dict(), "skipped_steps": self.skipped_steps}

    def load_state_dict(self, sd, load_optimizer_states=True):
        if load_optimizer_states and "optimizer_state_dict" in sd:
            self.optimizer.load_state_dict(sd["optimizer_state_dict"])
        self.skipped_steps = sd.get("skipped_steps", 0)
