"""Minimal stand-in for the `deepspeed` package, for the reference arm of bench.py only.

The reference training stack imports DeepSpeed at module scope and hands the model to
`deepspeed.initialize`.  DeepSpeed is not installable offline, so this package re-provides, in plain
PyTorch + torch.distributed (NCCL), only the symbols the reference touches on its training path:

  init_distributed, initialize (-> an engine with backward/step/train_batch), zero.Init,
  checkpointing.{configure, checkpoint, get_cuda_rng_tracker, model_parallel_cuda_manual_seed},
  pipe.{PipelineModule, LayerSpec, TiedLayerSpec}, runtime.pipe.topology, moe.layer.MoE (import
  stub), ops.adam.FusedAdam (torch fused AdamW), launcher.runner helpers.

It imports nothing from gpt_neox_b200 and loads none of its native libraries: the model, the
tensor-parallel layers, the attention path and the loss that run under it are the stock reference.
Only the engine (mixed-precision optimizer wrapper, gradient accumulation, data-parallel gradient
reduction, 1F1B pipeline schedule) is this stand-in.
"""
import os

import torch
import torch.distributed as dist

from .runtime.activation_checkpointing import checkpointing          # noqa: F401
from .runtime.engine import ShimEngine
from .runtime.pipe.engine import ShimPipelineEngine
from . import zero, pipe, comm, moe, ops                                # noqa: F401

__version__ = "0.0-shim"


def init_distributed(dist_backend="nccl", auto_mpi_discovery=True, distributed_port=29500, verbose=True,
                     timeout=None, init_method=None, dist_init_required=None, **_):
    if dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", str(distributed_port))
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    kw = {}
    if timeout is not None:
        kw["timeout"] = timeout
    dist.init_process_group(backend=dist_backend, **kw)


def initialize(args=None, model=None, optimizer=None, model_parameters=None, training_data=None,
               lr_scheduler=None, mpu=None, dist_init_required=None, collate_fn=None, config=None,
               config_params=None):
    cfg = dict(config or config_params or getattr(args, "deepspeed_config", None) or {})
    if "gradient_clipping" not in cfg and getattr(args, "gradient_clipping", None):
        cfg["gradient_clipping"] = args.gradient_clipping
    if isinstance(model, pipe.PipelineModule):
        engine = ShimPipelineEngine(model, optimizer, lr_scheduler, cfg, model_parameters)
    else:
        engine = ShimEngine(model, optimizer, lr_scheduler, cfg, mpu, model_parameters)
    return engine, engine.optimizer, None, engine.lr_scheduler
