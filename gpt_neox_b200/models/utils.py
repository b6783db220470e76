"""Parameter grouping and sequence-parallel gradient synchronisation
(reference ``megatron/model/utils.py:30-74, 365-404``)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..parallel import mpu
from .norms import LayerNorm, RMSNorm, ScaleNorm

_NORMS = (LayerNorm, RMSNorm, ScaleNorm, torch.nn.LayerNorm)


def get_params_for_weight_decay_optimization(module, neox_args):
    """Two groups: decayed weights, and (norm params, every ``bias``, params flagged
    ``_no_weight_decay``) without decay.  A single group is returned when weight decay is 0."""
    decay = {"params": [], "name": "weight_decay_params"}
    no_decay = {"params": [], "weight_decay": 0.0, "name": "no_weight_decay_params"}

    def skip(name, p):
        return name == "bias" or getattr(p, "_no_weight_decay", False)

    for m in module.modules():
        if isinstance(m, _NORMS) or neox_args.weight_decay == 0.0:
            no_decay["params"].extend(p for p in m._parameters.values() if p is not None)
        else:
            decay["params"].extend(p for n, p in m._parameters.items() if p is not None and not skip(n, p))
            no_decay["params"].extend(p for n, p in m._parameters.items() if p is not None and skip(n, p))
    if neox_args.weight_decay == 0.0:
        return [no_decay]
    return decay, no_decay


def norm_parameters(module):
    """Parameters replicated across a tensor-parallel group whose gradients are computed on a
    sequence shard only (all norm gains / biases, incl. per-head qk norms)."""
    out = []
    for name, p in module.named_parameters():
        if p.requires_grad and ("norm" in name.lower() or getattr(p, "sequence_parallel_grad_sync", False)):
            out.append(p)
    return out


def mark_norms_for_sequence_parallel_grad_sync(module, neox_args):
    """Under sequence parallelism each TP rank sees only its sequence shard inside norms, so their
    gradients must be summed over the TP group.  The reference installs one all-reduce hook per
    parameter (many tiny messages); here the parameters are only *tagged* and the engine reduces all
    of them in one flattened all-reduce after backward."""
    if not neox_args.sequence_parallel or mpu.get_model_parallel_world_size() == 1:
        return []
    params = norm_parameters(module)
    for p in params:
        p.sequence_parallel_grad_sync = True
        p.late_grad_sync = True        # rewritten after backward: not part of an early data-parallel reduction
    return params


def reduce_sequence_parallel_grads(params):
    """One flattened all-reduce over the TP group for all tagged parameters."""
    if not params or mpu.get_model_parallel_world_size() == 1:
        return
    grads = []
    for p in params:
        g = getattr(p, "main_grad", None)
        if g is None:
            g = p.grad
        if g is not None:
            grads.append(g)
    if not grads:
        return
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    for gs in by_dtype.values():
        flat = torch.cat([g.reshape(-1) for g in gs])
        dist.all_reduce(flat, group=mpu.get_model_parallel_group())
        off = 0
        for g in gs:
            g.copy_(flat[off:off + g.numel()].view_as(g))
            off += g.numel()
