"""Floating-point-operation counter fed by the kernel front-ends (``ops.gemm.gemm``, ``ops.fp8.gemm_fp8``, the eager
linear fallback, the attention entry points) and read by ``utils.flops_profiler.FlopsProfiler``.  Inactive (one
``is None`` test per call) unless a profiler is counting."""
from __future__ import annotations

ACTIVE = [None]     # the object whose ``flops`` attribute is being incremented, if any


def add(n):
    sink = ACTIVE[0]
    if sink is not None and sink.counting:
        sink.flops += n


def gemm(M, N, K):
    if ACTIVE[0] is not None:
        add(2.0 * M * N * K)


def attention(batch, heads, sq, sk, d, causal):
    if ACTIVE[0] is not None:
        add(4.0 * batch * heads * sq * sk * d * (0.5 if causal and sq == sk else 1.0))
