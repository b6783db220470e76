"""Vocabulary-parallel cross entropy.

Each tensor-parallel rank holds a contiguous slice ``[v0, v1)`` of the vocabulary dimension of the
logits.  Math (reference ``megatron/mpu/cross_entropy.py:27-117``): subtract the global row max,
gather the target logit from whichever rank owns it, sum the exponentials globally,
``loss = log(sum_exp) - target_logit``; backward is ``softmax - onehot``.

Differences in mechanism, not in math: the reference issues three all-reduces (max, target logit,
sum-exp) and keeps the full softmax alive for backward; here the target logit and the sum-exp travel
in ONE all-reduce of a ``[rows, 2]`` tensor, only two fp32 scalars per row are saved, and the
softmax is re-formed in backward directly into the gradient buffer.  On CUDA the row statistics
and the backward are single-pass kernels (the ``ce_*`` kernels of
``ops/csrc/misc_kernels.cu``).
"""
from __future__ import annotations


import torch
import torch.distributed as dist

from ..ops import native
from ..ops.functional import _DT, _k, _s
from . import mpu


def _row_stats(logits2, target, v0, row_max):
    """Per row: sum of exp(x - row_max) over the local slice and the (shifted) target logit if owned."""
    rows, vloc = logits2.shape
    if _k(logits2):
        stats = torch.empty(rows, 2, dtype=torch.float32, device=logits2.device)
        rc = native.lib().neox_ce_stats(native.ptr(logits2), native.ptr(target), native.ptr(row_max),
                                        native.ptr(stats), rows, vloc, v0, _DT[logits2.dtype], _s())
        native.check(rc, "neox_ce_stats")
        return stats
    xf = logits2.float() - row_max[:, None]
    sum_exp = xf.exp().sum(-1)
    local_t = target - v0
    owned = (local_t >= 0) & (local_t < vloc)
    idx = local_t.clamp(0, vloc - 1)
    pred = xf.gather(1, idx[:, None]).squeeze(1) * owned
    return torch.stack([sum_exp, pred], dim=1)


def _row_max(logits2):
    if _k(logits2):
        out = torch.empty(logits2.shape[0], dtype=torch.float32, device=logits2.device)
        rc = native.lib().neox_row_max(native.ptr(logits2), native.ptr(out), logits2.shape[0], logits2.shape[1],
                                       _DT[logits2.dtype], _s())
        native.check(rc, "neox_row_max")
        return out
    return logits2.float().max(-1).values


class _VocabParallelCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, logits, target):
        vloc = logits.shape[-1]
        logits2 = logits.reshape(-1, vloc)
        if not logits2.is_contiguous():
            logits2 = logits2.contiguous()
        tgt = target.reshape(-1).contiguous()
        tp = mpu.get_model_parallel_world_size()
        v0 = mpu.get_model_parallel_rank() * vloc
        if _k(logits2) and logits2.dtype == torch.bfloat16 and vloc % 8 == 0 and \
                native.lib().has("neox_ce_online_bf16"):
            # one pass over the logits: local (max, sum exp, raw target logit), re-based on the global maximum after
            # the first all-reduce
            rows = logits2.shape[0]
            row_max = torch.empty(rows, dtype=torch.float32, device=logits2.device)
            stats = torch.empty(rows, 2, dtype=torch.float32, device=logits2.device)
            rc = native.lib().neox_ce_online_bf16(native.ptr(logits2), native.ptr(tgt), native.ptr(row_max),
                                                  native.ptr(stats), rows, vloc, v0, _s())
            native.check(rc, "neox_ce_online_bf16")
            local_max = row_max
            if tp > 1:
                row_max = local_max.clone()
                dist.all_reduce(row_max, op=dist.ReduceOp.MAX, group=mpu.get_model_parallel_group())
                stats[:, 0] *= torch.exp(local_max - row_max)
            local_t = tgt - v0
            owned = (local_t >= 0) & (local_t < vloc)
            stats[:, 1] = torch.where(owned, stats[:, 1] - row_max, torch.zeros_like(row_max))
        else:
            row_max = _row_max(logits2)
            if tp > 1:
                dist.all_reduce(row_max, op=dist.ReduceOp.MAX, group=mpu.get_model_parallel_group())
            stats = _row_stats(logits2, tgt, v0, row_max)
        if tp > 1:
            dist.all_reduce(stats, group=mpu.get_model_parallel_group())
        loss = torch.log(stats[:, 0]) - stats[:, 1]
        ctx.save_for_backward(logits2, tgt, row_max, stats)
        ctx.v0 = v0
        ctx.shape = logits.shape
        return loss.reshape(target.shape)

    @staticmethod
    def backward(ctx, g):
        logits2, tgt, row_max, stats = ctx.saved_tensors
        rows, vloc = logits2.shape
        g1 = g.reshape(-1).float().contiguous()
        if _k(logits2):
            grad = torch.empty_like(logits2)
            rc = native.lib().neox_ce_bwd(native.ptr(logits2), native.ptr(tgt), native.ptr(row_max),
                                          native.ptr(stats), native.ptr(g1), native.ptr(grad), rows, vloc, ctx.v0,
                                          _DT[logits2.dtype], _s())
            native.check(rc, "neox_ce_bwd")
        else:
            sm = (logits2.float() - row_max[:, None]).exp() / stats[:, 0:1]
            local_t = tgt - ctx.v0
            owned = (local_t >= 0) & (local_t < vloc)
            idx = local_t.clamp(0, vloc - 1)
            sm[torch.arange(rows, device=sm.device), idx] -= owned.float()
            grad = (sm * g1[:, None]).to(logits2.dtype)
        return grad.reshape(ctx.shape), None


def vocab_parallel_cross_entropy(vocab_parallel_logits, target):
    """Per-token loss, shape of ``target``.  Logits may be bf16/fp16/fp32; statistics are fp32."""
    return _VocabParallelCE.apply(vocab_parallel_logits, target)
