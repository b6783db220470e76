"""Gradient noise scale (McCandlish et al. 2018, "An Empirical Model of Large-Batch Training").

B_simple ~= tr(Sigma) / |G|^2 is estimated from gradient norms at two batch sizes: every step gives a
"small batch" gradient (norm |G_small|), and the running mean of ``n_batches`` consecutive steps gives a
"big batch" gradient (norm |G_big|)::

    |G|^2     ~= (B_big |G_big|^2 - B_small |G_small|^2) / (B_big - B_small)
    tr(Sigma) ~= (|G_small|^2 - |G_big|^2) / (1/B_small - 1/B_big)

Both are smoothed by a bias-corrected EMA before taking the ratio.  Instead of copying every gradient tensor
each step (the reference keeps a full flattened copy, ``gradient_noise_scale.py:26-210``), this version reads
the engine's flat fp32 gradient buffers, which already are one contiguous vector per bucket, and keeps one
running-sum copy.  With pipeline parallelism the squared norms are summed over stages.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def ema(avg, beta, yi, i):
    """Bias-corrected exponential moving average: returns (new raw average, corrected value)."""
    if avg is None:
        avg = 0.0
    avg = beta * avg + (1 - beta) * yi
    return avg, avg / (1 - beta ** (i + 1))


class GradientNoiseScale:
    def __init__(self, model, batch_size_small, n_batches=10, beta=0.99, cpu_offload=False, neox_args=None, mpu=None):
        self.model = model
        self.batch_size_small = batch_size_small
        self.batch_size_large = batch_size_small * n_batches
        self.n_batches, self.beta, self.cpu_offload = n_batches, beta, cpu_offload
        self.neox_args, self.mpu = neox_args, mpu
        self.buffer = None
        self.ema_scale = self.ema_noise = self.noise_scale = None
        self.n_updates = 0
        self.model.store_gradients = True

    def flatten_grads(self):
        stored = getattr(self.model, "stored_gradients", None)
        if not stored:
            return None
        flat = torch.cat([g.reshape(-1).float() for g in stored if g is not None])
        if not torch.isfinite(flat).all():
            return None
        return flat.cpu() if self.cpu_offload else flat

    def _sync_overflow(self, is_overflow):
        if self.neox_args is not None and self.neox_args.is_pipe_parallel and dist.is_initialized():
            dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else "cpu"
            t = torch.tensor([int(is_overflow)], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.mpu.get_pipe_parallel_group())
            return bool(t.item())
        return is_overflow

    def _sq_norm(self, g):
        n = torch.square(torch.linalg.vector_norm(g))
        if self.neox_args is not None and self.neox_args.is_pipe_parallel and dist.is_initialized():
            n = n.to("cuda" if torch.cuda.is_available() else "cpu")
            dist.all_reduce(n, group=self.mpu.get_pipe_parallel_group())
        return n

    def _update(self):
        grad = self.flatten_grads()
        if self._sync_overflow(grad is None):
            return
        self.buffer = grad.clone() if self.buffer is None else self.buffer.add_(grad)
        if self.n_updates % self.n_batches == self.n_batches - 1:
            self.buffer /= self.n_batches
            g_big, g_small = self._sq_norm(self.buffer), self._sq_norm(grad)
            if bool(torch.isnan(g_big)) or bool(torch.isnan(g_small)):
                return
            g_big, g_small = float(g_big), float(g_small)
            noise = (g_small - g_big) / (1 / self.batch_size_small - 1 / self.batch_size_large)
            scale = (self.batch_size_large * g_big - self.batch_size_small * g_small) / \
                (self.batch_size_large - self.batch_size_small)
            i = self.n_updates // self.n_batches
            self.ema_noise, noise_c = ema(self.ema_noise, self.beta, noise, i)
            self.ema_scale, scale_c = ema(self.ema_scale, self.beta, scale, i)
            self.noise_scale = scale_c / noise_c if noise_c != 0 else None
            self.buffer = None
        self.n_updates += 1

    def update(self):
        if self.neox_args is not None and self.neox_args.is_pipe_parallel:
            self._update()
        else:
            if getattr(self.model, "micro_steps", 0) % getattr(self.model, "gas", 1) == 0:
                self._update()
