"""Process bootstrap: device selection, rendezvous, process groups, seeds, native helpers
(role of ``megatron/initialize.py:34-225``).

* backend ``nccl`` on GPUs, ``gloo`` when no GPU is present (or when asked for);
* device = ``local_rank`` (falls back to ``rank % device_count``);
* rank grid pipe -> data -> model, groups from ``parallel.mpu.initialize_model_parallel``;
* seeds: python / numpy / torch = ``seed``; interior pipeline stages draw from
  ``seed + 1138 + stage * mp`` so that they initialise different weights; the tensor-parallel RNG
  stream is ``seed + 2718 + tp_rank``.
"""
from __future__ import annotations

import datetime
import os
import random

import numpy as np
import torch
import torch.distributed as dist

from .parallel import mpu
from .parallel.rng import model_parallel_cuda_manual_seed
from .utils import print_rank_0


def _init_distributed(neox_args):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available()
    backend = neox_args.distributed_backend
    if not use_cuda and backend == "nccl":
        backend = "gloo"
    if use_cuda:
        n = torch.cuda.device_count()
        device = local if local < n else rank % n
        torch.cuda.set_device(device)
    if world > 1 or "MASTER_ADDR" in os.environ:
        if not dist.is_initialized():
            os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
            os.environ.setdefault("MASTER_PORT", str(getattr(neox_args, "master_port", None) or 6000))
            kwargs = {}
            if use_cuda and backend == "nccl":
                kwargs["device_id"] = torch.device("cuda", torch.cuda.current_device())
            dist.init_process_group(backend=backend, world_size=world, rank=rank,
                                    timeout=datetime.timedelta(minutes=30), **kwargs)
    neox_args.rank, neox_args.local_rank, neox_args.world_size = rank, local, world
    pp = max(neox_args.pipe_parallel_size, 1)
    mp = neox_args.model_parallel_size
    dp = world // (pp * mp)
    assert pp * mp * dp == world, f"world size {world} is not pp*mp*dp = {pp}*{mp}*{dp}"
    topo = mpu.Topology(pp=pp, dp=dp, mp=mp)
    mpu.initialize_model_parallel(mp, pp, expert_parallel_size=neox_args.moe_expert_parallel_size or 1, topology=topo,
                                  fp32_allreduce=neox_args.fp32_allreduce)
    return topo


def _set_random_seed(seed):
    if seed is None or seed <= 0:
        raise ValueError(f"Seed ({seed}) should be a positive integer.")
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    model_parallel_cuda_manual_seed(seed)


def initialize_megatron(neox_args, allow_no_cuda=False):
    """Idempotent set-up of distributed state, seeds and the native helper library."""
    if not mpu.model_parallel_is_initialized():
        _init_distributed(neox_args)
    seed = neox_args.seed
    if neox_args.pipe_parallel_size > 1 and mpu.get_pipe_parallel_world_size() > 1:
        stage = mpu.get_pipe_parallel_rank()
        if 0 < stage < mpu.get_pipe_parallel_world_size() - 1:
            seed = seed + 1138 + stage * mpu.get_model_parallel_world_size()
    if neox_args.rank == 0:
        print(f"> setting random seeds to {neox_args.seed} ...", flush=True)
    _set_random_seed(seed)
    # activation-checkpoint storage: sliced over the tensor-parallel group and / or parked in host memory.  Under
    # sequence parallelism the layer inputs are already per-rank shards, so there is nothing left to partition.
    from .parallel.rng import configure_checkpointing
    configure_checkpointing(bool(neox_args.partition_activations) and not bool(neox_args.sequence_parallel),
                            bool(neox_args.checkpoint_in_cpu))
    # build (local rank 0) and load the native libraries before any training step needs them
    from .ops import build as _build
    if neox_args.local_rank == 0:
        try:
            _build.build_host()
            if torch.cuda.is_available():
                _build.build_cuda()
        except Exception as exc:  # a missing compiler must not stop a run whose libraries are already built
            print_rank_0(f"native build skipped: {exc}")
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if torch.cuda.is_available():
        from .ops import native
        native.lib()
    return None
