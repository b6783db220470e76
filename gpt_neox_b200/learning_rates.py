"""Learning-rate schedule: linear warm-up, then constant / linear / cosine / exponential decay down to
``min_lr`` (behaviour of ``megatron/learning_rates.py:25-148``, including the checkpoint
``override_lr_scheduler`` / ``use_checkpoint_lr_scheduler`` semantics and muP per-group width scaling)."""
from __future__ import annotations

import math

_CURVES = {
    "linear": lambda t: 1.0 - t,
    "cosine": None,            # handled separately because it interpolates towards min_lr
    "exponential": lambda t: math.exp(-0.693 * t),
    "constant": lambda t: 1.0,
}


class AnnealingLR:
    _STATE = ("start_lr", "warmup_iter", "num_iters", "decay_style", "end_iter", "min_lr")

    def __init__(self, optimizer, start_lr, warmup_iter, total_iters, decay_style, last_iter, min_lr=0.0,
                 use_checkpoint_lr_scheduler=True, override_lr_scheduler=False, use_mup=False):
        assert total_iters > 0
        assert not (override_lr_scheduler and use_checkpoint_lr_scheduler), "both override and use-checkpoint are set."
        self.optimizer = optimizer
        self.start_lr, self.min_lr = start_lr, min_lr
        self.warmup_iter, self.end_iter, self.num_iters = warmup_iter, total_iters, last_iter
        self.decay_style = decay_style
        self.override_lr_scheduler = override_lr_scheduler
        self.use_checkpoint_lr_scheduler = use_checkpoint_lr_scheduler
        self.use_mup = use_mup
        self.step(self.num_iters)

    def get_lr(self):
        n = self.num_iters
        if self.warmup_iter > 0 and n <= self.warmup_iter:
            return float(self.start_lr) * n / self.warmup_iter
        span = self.end_iter - self.warmup_iter
        t = (n - self.warmup_iter) / span if span > 0 else 1.0
        if self.decay_style == "cosine":
            lr = self.min_lr + (self.start_lr - self.min_lr) / 2.0 * (math.cos(math.pi * t) + 1)
        else:
            lr = self.start_lr * _CURVES.get(self.decay_style, _CURVES["constant"])(t)
        return max(lr, self.min_lr)

    def step(self, step_num=None):
        self.num_iters = self.num_iters + 1 if step_num is None else step_num
        lr = self.get_lr()
        for group in self.optimizer.param_groups:
            group["lr"] = lr / group["width_mult"] if (self.use_mup and "width_mult" in group) else lr

    def state_dict(self):
        return {k: getattr(self, k) for k in self._STATE}

    def _resolve(self, mine, saved, what):
        if self.override_lr_scheduler:
            return mine
        if not self.use_checkpoint_lr_scheduler:
            assert mine == saved, f"AnnealingLR: class input value and checkpoint values for {what} do not match"
        return saved

    def load_state_dict(self, sd):
        for key in ("start_lr", "min_lr", "warmup_iter", "end_iter", "decay_style"):
            setattr(self, key, self._resolve(getattr(self, key), sd[key], key))
        self.step(sd["num_iters"])
