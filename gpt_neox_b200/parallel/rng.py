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


# How checkpointed inputs are kept between forward and backward (reference: the DeepSpeed activation-checkpointing
# options the reference forwards in ``megatron/initialize.py:89-118``):
#   partition   -- every tensor-parallel rank keeps only its 1/tp slice of each saved floating-point input and the
#                  slices are all-gathered over the TP group right before the recomputation (the inputs of a layer are
#                  replicated across TP ranks, so nothing is lost and activation memory drops by tp);
#   cpu         -- the kept (slice of the) tensor is parked in pinned host memory and copied back for the recomputation.
_CKPT_CFG = {"partition": False, "cpu": False}


def configure_checkpointing(partition_activations=False, checkpoint_in_cpu=False):
    _CKPT_CFG["partition"] = bool(partition_activations)
    _CKPT_CFG["cpu"] = bool(checkpoint_in_cpu)


def _stash(t):
    """(kept tensor, recipe to rebuild the original)."""
    from . import mpu
    tp = mpu.get_model_parallel_world_size() if mpu.model_parallel_is_initialized() else 1
    meta = {"shape": t.shape, "part": False, "cpu": False, "device": t.device, "req": t.requires_grad}
    keep = t
    if _CKPT_CFG["partition"] and tp > 1 and t.is_floating_point() and t.numel() % tp == 0 and t.numel() >= tp:
        r = mpu.get_model_parallel_rank()
        n = t.numel() // tp
        keep = t.detach().reshape(-1)[r * n:(r + 1) * n].clone()
        meta["part"] = True
    if _CKPT_CFG["cpu"] and keep.is_cuda:
        host = torch.empty(keep.shape, dtype=keep.dtype, device="cpu", pin_memory=True)
        host.copy_(keep.detach(), non_blocking=True)
        keep = host
        meta["cpu"] = True
    return keep, meta


def _unstash(keep, meta):
    import torch.distributed as dist
    from . import mpu
    t = keep
    if meta["cpu"]:
        t = t.to(meta["device"], non_blocking=True)
    if meta["part"]:
        tp = mpu.get_model_parallel_world_size()
        full = torch.empty(t.numel() * tp, dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(full, t.contiguous(), group=mpu.get_model_parallel_group())
        t = full.view(meta["shape"])
    return t


# While a checkpointed block is re-run in backward, the output of its LAST layer is never read: backward only needs
# what the ops saved (their inputs).  ``recompute_tail()`` tells that layer so, and it skips the GEMMs (and the
# tensor-parallel reduction) that produce nothing but that output.
_RECOMPUTE = {"active": False, "tail": False}


def in_recompute() -> bool:
    return _RECOMPUTE["active"]


def set_block_tail(is_last: bool):
    """Called by the layer runners before each layer of a block: is this the last layer of the block?"""
    _RECOMPUTE["tail"] = bool(is_last)


def recompute_tail() -> bool:
    """True inside the recomputation of the last layer of a checkpointed block (``NEOX_RECOMPUTE_SKIP_TAIL=0`` turns
    the short-cut off)."""
    if "enabled" not in _RECOMPUTE:
        import os
        _RECOMPUTE["enabled"] = os.environ.get("NEOX_RECOMPUTE_SKIP_TAIL", "1") != "0"
    return _RECOMPUTE["active"] and _RECOMPUTE["tail"] and _RECOMPUTE["enabled"]


def set_recompute_skip(enabled: bool):
    _RECOMPUTE["enabled"] = bool(enabled)


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
        tensors = [a for a in args if torch.is_tensor(a)]
        if _CKPT_CFG["partition"] or _CKPT_CFG["cpu"]:
            kept = [_stash(t) for t in tensors]
            ctx.metas = [m for _, m in kept]
            ctx.save_for_backward(*[k for k, _ in kept])
        else:
            ctx.metas = None
            ctx.save_for_backward(*tensors)
        with torch.no_grad():
            out = fn(*args)
        return out

    @staticmethod
    def backward(ctx, *grads):
        saved = list(ctx.saved_tensors)
        if ctx.metas is not None:
            reqs = [m["req"] for m in ctx.metas]
            saved = [_unstash(k, m) for k, m in zip(saved, ctx.metas)]
        else:
            reqs = [t.requires_grad for t in saved]
        args, it, rq = [], iter(saved), iter(reqs)
        for is_t, c in zip(ctx.is_tensor, ctx.consts):
            if is_t:
                t = next(it)
                d = t.detach()
                d.requires_grad_(next(rq))
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
        _RECOMPUTE["active"] = True
        try:
            with torch.enable_grad():
                out = ctx.fn(*args)
        finally:
            _RECOMPUTE["active"] = False
            _RECOMPUTE["tail"] = False
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
