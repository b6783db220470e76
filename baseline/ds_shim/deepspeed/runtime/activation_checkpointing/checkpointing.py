"""Activation checkpointing with a named CUDA RNG-state tracker (Megatron semantics).

`checkpoint(fn, *args)` runs fn without building a graph, remembers the CPU / CUDA / tracker RNG
states, and re-runs fn under those states in backward.  `model_parallel_cuda_manual_seed(seed)` gives
the default CUDA generator the same stream on all tensor-parallel ranks and registers a
"model-parallel-rng" stream that differs per tensor-parallel rank.
"""
import contextlib

import torch

_MODEL_PARALLEL_RNG_TRACKER_NAME = "model-parallel-rng"
_mpu = None
_cfg = {}


def _set_cuda_rng_state(state, device=-1):
    if device == -1:
        device = torch.cuda.current_device()
    torch.cuda.set_rng_state(state, device)


class CudaRNGStatesTracker:
    def __init__(self):
        self.reset()

    def reset(self):
        self.states_, self.seeds_ = {}, set()

    def get_states(self):
        return dict(self.states_)

    def set_states(self, states):
        self.states_ = states

    def add(self, name, seed):
        if seed in self.seeds_:
            raise Exception(f"seed {seed} already exists")
        if name in self.states_:
            raise Exception(f"cuda rng state {name} already exists")
        self.seeds_.add(seed)
        keep = torch.cuda.get_rng_state()
        torch.cuda.manual_seed(seed)
        self.states_[name] = torch.cuda.get_rng_state()
        _set_cuda_rng_state(keep)

    @contextlib.contextmanager
    def fork(self, name=_MODEL_PARALLEL_RNG_TRACKER_NAME):
        if name not in self.states_:
            raise Exception(f"cuda rng state {name} is not added")
        keep = torch.cuda.get_rng_state()
        _set_cuda_rng_state(self.states_[name])
        try:
            yield
        finally:
            self.states_[name] = torch.cuda.get_rng_state()
            _set_cuda_rng_state(keep)


_CUDA_RNG_STATE_TRACKER = CudaRNGStatesTracker()


def get_cuda_rng_tracker():
    return _CUDA_RNG_STATE_TRACKER


def model_parallel_cuda_manual_seed(seed):
    tp_rank = _mpu.get_model_parallel_rank() if _mpu is not None else 0
    _CUDA_RNG_STATE_TRACKER.reset()
    torch.cuda.manual_seed(seed)
    _CUDA_RNG_STATE_TRACKER.add(_MODEL_PARALLEL_RNG_TRACKER_NAME, seed + 2718 + tp_rank)


def configure(mpu_, deepspeed_config=None, partition_activations=None, contiguous_checkpointing=None,
              num_checkpoints=None, checkpoint_in_cpu=None, synchronize=None, profile=None):
    global _mpu
    _mpu = mpu_
    _cfg.update(partition_activations=partition_activations, checkpoint_in_cpu=checkpoint_in_cpu,
                synchronize=synchronize)


def is_configured():
    return _mpu is not None


def reset():
    pass


class _Checkpoint(torch.autograd.Function):
    @staticmethod
    def forward(ctx, fn, n_tensor_out_holder, *args):
        ctx.fn = fn
        ctx.cpu_rng = torch.get_rng_state()
        ctx.cuda_rng = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        ctx.tracker = get_cuda_rng_tracker().get_states()
        ctx.is_tensor = [torch.is_tensor(a) for a in args]
        ctx.save_for_backward(*[a for a in args if torch.is_tensor(a)])
        ctx.others = [a for a in args if not torch.is_tensor(a)]
        with torch.no_grad():
            out = fn(*args)
        ctx.single = torch.is_tensor(out)
        outs = (out,) if ctx.single else tuple(out)
        non_diff = [o for o in outs if torch.is_tensor(o) and not o.is_floating_point()]
        ctx.mark_non_differentiable(*non_diff)
        return out if ctx.single else outs

    @staticmethod
    def backward(ctx, *grads):
        saved, others = list(ctx.saved_tensors), list(ctx.others)
        args = []
        for t in ctx.is_tensor:
            if t:
                a = saved.pop(0)
                d = a.detach()
                d.requires_grad = a.requires_grad
                args.append(d)
            else:
                args.append(others.pop(0))
        keep_cpu = torch.get_rng_state()
        keep_cuda = torch.cuda.get_rng_state() if ctx.cuda_rng is not None else None
        keep_tr = get_cuda_rng_tracker().get_states()
        torch.set_rng_state(ctx.cpu_rng)
        if ctx.cuda_rng is not None:
            _set_cuda_rng_state(ctx.cuda_rng)
        get_cuda_rng_tracker().set_states(ctx.tracker)
        with torch.enable_grad():
            out = ctx.fn(*args)
        torch.set_rng_state(keep_cpu)
        if keep_cuda is not None:
            _set_cuda_rng_state(keep_cuda)
        get_cuda_rng_tracker().set_states(keep_tr)
        outs = (out,) if torch.is_tensor(out) else tuple(out)
        pairs = [(o, g) for o, g in zip(outs, grads) if torch.is_tensor(o) and o.requires_grad and g is not None]
        torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])
        return (None, None) + tuple(a.grad if torch.is_tensor(a) and a.requires_grad else None for a in args)


def checkpoint(function, *args):
    return _Checkpoint.apply(function, None, *args)
