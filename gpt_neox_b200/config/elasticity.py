"""Elastic batch configuration: one global batch size that stays valid while the number of GPUs changes.

The reference passes its ``elasticity`` block (``enabled, max_train_batch_size, micro_batch_sizes, min_gpus, max_gpus,
prefer_larger_batch, ignore_non_elastic_batch_info``; ``megatron/neox_arguments/deepspeed_args.py:229``) to DeepSpeed,
which at start-up replaces the configured batch triple by an "elastic" one.  This module computes the same kind of
answer: among all global batch sizes up to ``max_train_batch_size`` that some allowed micro-batch divides, take the
one that can be split evenly over the largest number of different GPU counts in ``[min_gpus, max_gpus]`` (ties: the
larger batch when ``prefer_larger_batch``), then for the GPU count actually present pick the largest allowed
micro-batch that divides the per-GPU share; the remainder becomes gradient accumulation steps.
"""
from __future__ import annotations


class ElasticityError(ValueError):
    pass


def valid_gpu_counts(batch, micro_batches, min_gpus, max_gpus):
    """GPU counts that can run ``batch`` with one of the allowed micro-batch sizes and whole accumulation steps."""
    return [g for g in range(min_gpus, max_gpus + 1) if any(batch % (mb * g) == 0 for mb in micro_batches)]


def compute_elastic_config(block, world_size=None):
    """``(train_batch_size, valid_gpus, micro_batch)``; ``micro_batch`` is ``None`` when ``world_size`` is ``None``.
    Raises ``ElasticityError`` when no batch fits or the present GPU count cannot run the chosen batch."""
    micro = sorted({int(m) for m in block.get("micro_batch_sizes", [])})
    if not micro or any(m <= 0 for m in micro):
        raise ElasticityError("elasticity.micro_batch_sizes must list positive micro-batch sizes")
    max_batch = int(block.get("max_train_batch_size", 0))
    if max_batch < micro[0]:
        raise ElasticityError(f"elasticity.max_train_batch_size ({max_batch}) is smaller than every micro-batch size")
    min_gpus = int(block.get("min_gpus", 1))
    max_gpus = int(block.get("max_gpus", max(max_batch // micro[0], 1)))
    if min_gpus < 1 or max_gpus < min_gpus:
        raise ElasticityError(f"invalid elasticity GPU range [{min_gpus}, {max_gpus}]")
    prefer_larger = bool(block.get("prefer_larger_batch", True))
    best = None
    candidates = sorted({b for mb in micro for b in range(mb, max_batch + 1, mb)})
    for batch in candidates:
        gpus = valid_gpu_counts(batch, micro, min_gpus, max_gpus)
        if not gpus:
            continue
        key = (len(gpus), batch if prefer_larger else -batch)
        if best is None or key > best[0]:
            best = (key, batch, gpus)
    if best is None:
        raise ElasticityError("no batch size up to max_train_batch_size fits any GPU count in the elastic range")
    _, batch, gpus = best
    micro_batch = None
    if world_size is not None:
        if world_size not in gpus:
            raise ElasticityError(f"the elastic batch size {batch} cannot be split over {world_size} GPUs "
                                  f"(valid counts: {gpus})")
        micro_batch = max(mb for mb in micro if batch % (mb * world_size) == 0)
    return batch, gpus, micro_batch
