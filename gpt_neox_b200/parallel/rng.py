"""Model-parallel random-number streams and activation checkpointing.

The reference delegates both to DeepSpeed (``megatron/mpu/random.py:18-37``):

* a *tracker* that owns named RNG states -- ``model-parallel-rng`` differs per tensor-parallel rank
  (used for dropout inside TP regions and for initialising sharded weights,
  ``megatron/mpu/layers.py:51-52``, ``megatron/model/transformer.py:592-593``) while the default
  stream is identical across a TP group;
* ``checkpoint(fn, *args)``: run ``fn`` without storing activations and replay it in backward with
  exactly the RNG states of the first run.

Both are implemented here on top of plain ``torch`` generators so they work on CPU and CUDA.
"""
from __future__ import annotations

import contextlib

import torch

from . import mpu

_MODEL_PARALLEL_RNG = "model-parallel-rng"


def _get_state(device_is_cuda):
    return torch.cuda.get_rng_state() if device_is_cuda else torch.get_rng_state()


def _set_state(state, device_is_cuda):
    if device_is_cuda:
        torch.cuda.set_rng_state(state)
    else:
        torch.set_rng_state(state)


class RNGStatesTracker:
    """Named RNG states that can be temporarily swapped in with ``fork``."""

    def __init__(self):
        self.states = {}
        self.seeds = set()

    def reset(self):
        self.states, self.seeds = {}, set()

    def get_states(self):
        return dict(self.states)

    def set_states(self, states):
        self.states = dict(states)

    def add(self, name, seed):
        if seed in self.seeds:
            raise RuntimeError(f"seed {seed} already exists")
        if name in self.states:
            raise RuntimeError(f"rng state {name} already exists")
        self.seeds.add(seed)
        cuda = torch.cuda.is_available()
        saved = _get_state(cuda)
        if cuda:
            torch.cuda.manual_seed(seed)
        else:
            torch.manual_seed(seed)
        self.states[name] = _get_state(cuda)
        _set_state(saved, cuda)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG):
        if name not in self.states:
            # tracker never seeded (e.g. unit tests building a bare layer): behave as a no-op
            yield
            return
        cuda = torch.cuda.is_available()
        saved = _get_state(cuda)
        _set_state(self.states[name], cuda)
        try:
            yield
        finally:
            self.states[name] = _get_state(cuda)
            _set_state(saved, cuda)


_TRACKER = RNGStatesTracker()


def get_cuda_rng_tracker() -> RNGStatesTracker:
    return _TRACKER


def model_parallel_cuda_manual_seed(seed: int):
    """Default stream: ``seed`` (same on every TP rank); tracked TP stream: ``seed + 2718 + tp_rank``."""
    tp_seed = seed + 2718 + mpu.get_model_parallel_rank()
    _TRACKER.reset()
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)
    _TRACKER.add(_MODEL_PARALLEL_RNG, tp_seed)


class _Checkpoint(torch.autograd.Function):
    """Recompute-in-backward with RNG replay (default stream, CUDA stream and tracker states)."""

    @staticmethod
    def forward(ctx, fn, n_tensor, *args):
        ctx.fn = fn
        ctx.cpu_state = torch.get_rng_state()
        ctx.cuda_state = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        ctx.tracker_states = _TRACKER.get_states()
        ctx.is_tensor = [torch.is_tensor(a) for a in args]
        ctx.consts = [None if t else a for a, t in zip(args, ctx.is_tensor)]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        with torch.no_grad():
            out = fn(*args)
        return out

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        args, it = [], iter(saved)
        for is_t, c in zip(ctx.is_tensor, ctx.consts):
            if is_t:
                t = next(it)
                d = t.detach()
                d.requires_grad_(t.requires_grad)
                args.append(d)
            else:
                args.append(c)
        # replay under the RNG states of the first run, then restore the current ones
        cur_cpu = torch.get_rng_state()
        cur_cuda = torch.cuda.get_rng_state() if ctx.cuda_state is not None else None
        cur_tracker = _TRACKER.get_states()
        torch.set_rng_state(ctx.cpu_state)
        if ctx.cuda_state is not None:
            torch.cuda.set_rng_state(ctx.cuda_state)
        _TRACKER.set_states(ctx.tracker_states)
        with torch.enable_grad():
            out = ctx.fn(*args)
        torch.set_rng_state(cur_cpu)
        if cur_cuda is not None:
            torch.cuda.set_rng_state(cur_cuda)
        _TRACKER.set_states(cur_tracker)
        outs = out if isinstance(out, (tuple, list)) else (out,)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        if pairs:
            torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        result = [None, None]
        for a, is_t in zip(args, ctx.is_tensor):
            result.append(a.grad if is_t and torch.is_tensor(a) else None)
        return tuple(result)


def checkpoint(fn, *args):
    """Run ``fn(*args)`` without keeping its internal activations; recompute them in backward."""
    return _Checkpoint.apply(fn, len(args), *args)
