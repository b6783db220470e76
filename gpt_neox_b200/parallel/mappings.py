"""Tensor- and sequence-parallel region mappings as autograd functions.

Each mapping pairs a forward collective with its conjugate in backward
(reference: ``megatron/mpu/mappings.py:189-344``):

======================================  =====================  =====================
function                                forward                backward
======================================  =====================  =====================
copy_to_model_parallel_region           identity               all-reduce
reduce_from_model_parallel_region       all-reduce             identity
scatter_to_model_parallel_region        split last dim         all-gather last dim
gather_from_model_parallel_region       all-gather last dim    split last dim
reduce_scatter_to_sequence_parallel     reduce-scatter seq     all-gather seq
gather_from_sequence_parallel_region    all-gather seq         reduce-scatter seq
scatter_to_sequence_parallel_region     split seq              all-gather seq
======================================  =====================  =====================

All are the identity when the tensor-parallel world size is 1.  ``fp32_allreduce`` up-casts bf16
payloads for reductions.  These NCCL forms are the portable baseline; on B200 the linear layers
replace "all-gather -> GEMM" and "GEMM -> reduce-scatter" by fused peer-memory kernels
(``parallel/fused_comm.py``).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import mpu


def _tp():
    return mpu.get_model_parallel_world_size()


def _reduce(x):
    if _tp() == 1:
        return x
    x = x.contiguous()
    if mpu.get_fp32_allreduce() and x.dtype == torch.bfloat16:
        y = x.float()
        dist.all_reduce(y, group=mpu.get_model_parallel_group())
        return y.to(torch.bfloat16)
    dist.all_reduce(x, group=mpu.get_model_parallel_group())
    return x


def _split_last(x):
    if _tp() == 1:
        return x
    parts = mpu.split_tensor_along_last_dim(x, _tp())
    return parts[mpu.get_model_parallel_rank()].contiguous()


def _gather_last(x):
    n = _tp()
    if n == 1:
        return x
    x = x.contiguous()
    out = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(out, x, group=mpu.get_model_parallel_group())
    return torch.cat(out, dim=-1).contiguous()


def _reduce_scatter_seq(x, seq_dim):
    n = _tp()
    if n == 1:
        return x
    upcast = mpu.get_fp32_allreduce() and x.dtype == torch.bfloat16
    src = x.float() if upcast else x
    assert src.shape[seq_dim] % n == 0, f"sequence dim {src.shape[seq_dim]} not divisible by TP {n}"
    if seq_dim == 0:
        src = src.contiguous()
        out = torch.empty((src.shape[0] // n, *src.shape[1:]), dtype=src.dtype, device=src.device)
        dist.reduce_scatter_tensor(out, src, group=mpu.get_model_parallel_group())
    else:
        chunks = [c.contiguous() for c in torch.chunk(src, n, dim=seq_dim)]
        out = torch.empty_like(chunks[0])
        dist.reduce_scatter(out, chunks, group=mpu.get_model_parallel_group())
    return out.to(torch.bfloat16) if upcast else out


def _gather_seq(x, seq_dim):
    n = _tp()
    if n == 1:
        return x
    x = x.contiguous()
    if seq_dim == 0:
        out = torch.empty((x.shape[0] * n, *x.shape[1:]), dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=mpu.get_model_parallel_group())
        return out
    parts = [torch.empty_like(x) for _ in range(n)]
    dist.all_gather(parts, x, group=mpu.get_model_parallel_group())
    return torch.cat(parts, dim=seq_dim).contiguous()


def _split_seq(x, seq_dim):
    n = _tp()
    if n == 1:
        return x
    assert x.shape[seq_dim] % n == 0
    return torch.chunk(x, n, dim=seq_dim)[mpu.get_model_parallel_rank()].contiguous()


class _Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _reduce(g)


class _Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _reduce(x)

    @staticmethod
    def backward(ctx, g):
        return g


class _Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _split_last(x)

    @staticmethod
    def backward(ctx, g):
        return _gather_last(g)


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _gather_last(x)

    @staticmethod
    def backward(ctx, g):
        return _split_last(g)


class _ReduceScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim, values_unused=False):
        ctx.seq_dim = seq_dim
        if values_unused:
            # shape and autograd edge only (backward still all-gathers): the result of a recomputed block tail
            world = mpu.get_model_parallel_world_size()
            return x.narrow(seq_dim, 0, x.shape[seq_dim] // world).contiguous()
        return _reduce_scatter_seq(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.seq_dim), None, None


class _GatherSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _gather_seq(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_seq(g, ctx.seq_dim), None


class _ScatterSeq(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, seq_dim):
        ctx.seq_dim = seq_dim
        return _split_seq(x, seq_dim)

    @staticmethod
    def backward(ctx, g):
        return _gather_seq(g, ctx.seq_dim), None


def copy_to_model_parallel_region(x):
    return _Copy.apply(x)


def reduce_from_model_parallel_region(x):
    return _Reduce.apply(x)


def scatter_to_model_parallel_region(x):
    return _Scatter.apply(x)


def gather_from_model_parallel_region(x):
    return _Gather.apply(x)


def reduce_scatter_to_sequence_parallel_region(x, seq_dim=0, values_unused=False):
    return _ReduceScatterSeq.apply(x, seq_dim, values_unused)


def gather_from_sequence_parallel_region(x, seq_dim=0):
    return _GatherSeq.apply(x, seq_dim)


def scatter_to_sequence_parallel_region(x, seq_dim=0):
    return _ScatterSeq.apply(x, seq_dim)
