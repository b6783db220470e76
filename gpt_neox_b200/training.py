"""Pre-training / fine-tuning orchestration (role of ``megatron/training.py``).

Public surface kept from the reference: ``pretrain``, ``setup_model_and_optimizer``, ``get_model``,
``get_optimizer``, ``get_learning_rate_scheduler``, ``get_batch`` / ``get_batch_pipe`` /
``get_batch_sequential``, ``forward_step``, ``backward_step``, ``train_step``, ``train``, ``evaluate``,
``evaluate_and_print_results``, ``is_save_iter``, ``update_iterations``.
"""
from __future__ import annotations

import contextlib
import math
import sys
from contextlib import nullcontext
from functools import partial

import torch
import torch.distributed as dist

from . import objectives as OBJ
from .checkpointing import load_checkpoint, save_checkpoint
from .data.data_utils import build_train_valid_test_data_loaders, shift_and_wrap_data_loaders
from .engine.engine import NeoXEngine, PipelineEngine
from .engine.flat_optimizer import FlatMixedPrecisionOptimizer
from .initialize import initialize_megatron
from .learning_rates import AnnealingLR
from .logging import tb_wandb_log, training_log
from .models import (GPT2ModelPipe, SoftEmbedding, cross_entropy, get_params_for_weight_decay_optimization,
                     mark_norms_for_sequence_parallel_grad_sync)
from .parallel import mpu
from .parallel.data import broadcast_data
from .parallel import comms_logger
from .utils.flops_profiler import FlopsProfiler
from .utils import (CharCounter, OverflowMonitor, Timers, get_ltor_masks_and_position_ids, get_noise_scale_logger,
                    get_total_params, print_rank_0, reduce_losses)


def _nvtx(neox_args, name):
    if neox_args.memory_profiling or neox_args.profile:
        return torch.cuda.nvtx.range(name) if torch.cuda.is_available() else nullcontext()
    return nullcontext()


# ------------------------------------------------------------------------------------ iteration bookkeeping
def update_iterations(neox_args, data_loaders):
    """Derive ``train_iters`` from ``train_epochs`` (length of the train loader x epochs, agreed over ranks)."""
    if neox_args.train_iters is not None or neox_args.train_epochs is None:
        return
    n = len(data_loaders["train"]) * neox_args.train_epochs if data_loaders.get("train") is not None else 0
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    t = torch.tensor([n], dtype=torch.long, device=dev)
    if dist.is_available() and dist.is_initialized():
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    neox_args.train_iters = int(t.item())
    print_rank_0(f"setting training iterations to {neox_args.train_iters}")


def is_save_iter(neox_args, iteration):
    """Linear: every ``checkpoint_factor`` iterations; log: at powers of ``checkpoint_factor``; plus
    ``extra_save_iters``."""
    if neox_args.extra_save_iters and iteration in neox_args.extra_save_iters:
        return True
    f = neox_args.checkpoint_factor
    if not f:
        return False
    if neox_args.checkpoint_scale == "linear":
        return iteration % f == 0
    if neox_args.checkpoint_scale == "log":
        if iteration <= 0 or f <= 1:
            return False
        power = 1
        while power < iteration + f:
            if int(power) == iteration:
                return True
            power *= f
        return False
    return False


# ------------------------------------------------------------------------------------ batches
def _get_batch(neox_args, tokenizer, keys, data, datatype, label_mask_zero=False):
    data_b = broadcast_data(keys, data, datatype)
    token_key = keys[0]
    label_key = keys[1] if len(keys) > 1 else None
    tokens_ = data_b[token_key].long()
    if label_key in data_b:
        lab = data_b[label_key].long()
        label_mask = (lab >= 0)[:, 1:].contiguous()
        labels = torch.where(lab >= 0, lab, torch.zeros_like(lab))[:, 1:].contiguous()
    else:
        label_mask = (tokens_ >= 0)[:, 1:].contiguous()
        labels = tokens_[:, 1:].contiguous()
        if label_mask_zero:
            labels = labels * label_mask
    tokens = tokens_[:, :-1].contiguous()
    attention_mask, loss_mask, position_ids = get_ltor_masks_and_position_ids(
        data=tokens, eod_token=neox_args.tokenizer.eod if neox_args.tokenizer is not None else -1,
        eod_mask_loss=neox_args.eod_mask_loss, sliding_window_width=neox_args.sliding_window_width)
    loss_mask = label_mask.to(loss_mask.dtype) * loss_mask
    return tokens, labels, loss_mask, attention_mask, position_ids


def _next_batch(data_iterator, neox_args):
    """``next(data_iterator)`` with the rank and iteration attached to any failure of the data pipeline (a worker
    exception, a corrupt index, an exhausted dataset), so that the one failing rank of a large job can be found."""
    if data_iterator is None:
        return None
    try:
        return next(data_iterator)
    except StopIteration:
        raise RuntimeError(f"data iterator exhausted on rank {neox_args.rank} at iteration "
                           f"{getattr(neox_args, 'iteration', '?')}") from None
    except Exception as exc:
        raise RuntimeError(f"data loader failed on rank {neox_args.rank} at iteration "
                           f"{getattr(neox_args, 'iteration', '?')}: {type(exc).__name__}: {exc}") from exc


def get_batch(neox_args, data_iterator):
    """One micro-batch for the sequential engine, shaped by ``train_impl``."""
    impl = neox_args.train_impl
    data = _next_batch(data_iterator, neox_args)
    dt = torch.int64
    if impl in ("normal", "kto"):
        keys = ["text", "label"] if neox_args.train_label_data_paths else ["text"]
        if impl == "kto":
            assert neox_args.train_micro_batch_size_per_gpu > 1, "For KTO training, the train_micro_batch_size_per_gpu must be greater than 1."
        tup = _get_batch(neox_args, neox_args.tokenizer, keys, data, dt, label_mask_zero=impl == "kto")
        if impl == "normal":
            return tup
        rw = broadcast_data(["reward"], data, torch.float)["reward"][:, :-1].contiguous()
        ref_logp = None
        if data is not None and "ref" in data or neox_args.precompute_model_name:
            ref_logp = broadcast_data(["ref"], data, torch.float)["ref"][:, :-1].contiguous()
        return tup + (rw, ref_logp)
    if impl == "reinforce":
        tup = _get_batch(neox_args, neox_args.tokenizer, ["text"], data, dt, label_mask_zero=True)
        rws = broadcast_data(["reward", "raw_reward"], data, torch.float)
        rw = rws["reward"].unsqueeze(-1).expand(-1, tup[0].shape[1]) if rws["reward"].dim() == 1 \
            else rws["reward"][:, :-1].contiguous()
        return tup + (rw, rws["raw_reward"])
    if impl in ("dpo", "rm"):
        pos_keys = ["pos", "pos_label"] if neox_args.pos_train_label_data_paths else ["pos"]
        neg_keys = ["neg", "neg_label"] if neox_args.neg_train_label_data_paths else ["neg"]
        pos = _get_batch(neox_args, neox_args.tokenizer, pos_keys, data, dt, label_mask_zero=True)
        neg = _get_batch(neox_args, neox_args.tokenizer, neg_keys, data, dt, label_mask_zero=True)
        ref_logp = None
        if neox_args.precompute_model_name:
            r = broadcast_data(["pos_ref", "neg_ref"], data, torch.float)
            ref_logp = torch.cat((r["pos_ref"], r["neg_ref"]), dim=0)[:, :-1].contiguous()
        tokens = torch.cat((pos[0], neg[0]), 0)
        labels = torch.cat((pos[1], neg[1]), 0)
        loss_mask = torch.cat((pos[2], neg[2]), 0)
        position_ids = torch.cat((pos[4], neg[4]), 0)
        return tokens, labels, loss_mask, pos[3], position_ids, ref_logp
    raise ValueError(f"unknown train_impl {impl}")


def get_batch_pipe(data, neox_args, curr_scheduler=None):
    """Micro-batch for the pipeline engine: ``((tokens, position_ids, attention_mask), (labels, loss_mask))``."""
    assert neox_args.train_impl not in ("kto", "dpo", "rm"), "Pipeline parallel is currently unsupported when using any of kto, dpo, rm. Set pipe_parallel_size to 0"
    keys = ["text", "label"] if neox_args.train_label_data_paths else ["text"]
    tokens, labels, loss_mask, attention_mask, position_ids = _get_batch(neox_args, neox_args.tokenizer, keys, data,
                                                                         torch.int64)
    if curr_scheduler is not None:
        cur = curr_scheduler.update_difficulty(neox_args.iteration + 1) if neox_args.iteration is not None \
            else curr_scheduler.get_current_difficulty()
        if cur < tokens.size(1):
            tokens, position_ids, labels, loss_mask = (t[:, :cur].contiguous() for t in
                                                       (tokens, position_ids, labels, loss_mask))
            if attention_mask is not None:
                attention_mask = attention_mask[:, :, :cur, :cur].contiguous()
    return (tokens, position_ids, attention_mask), (labels, loss_mask)


def get_batch_sequential(forward_input, neox_args):
    """Rebuild mask / position ids from raw tokens (batch_fn of the sequential wrapper)."""
    attention_mask, _, position_ids = get_ltor_masks_and_position_ids(
        data=forward_input[0], eod_token=neox_args.tokenizer.eod, eod_mask_loss=neox_args.eod_mask_loss)
    return forward_input[0], forward_input[1], attention_mask


def mb_moe_loss_func(neox_args, moe_losses):
    """Load-balancing auxiliary loss: mean over MoE layers of the per-layer losses the routers returned
    (each already ``num_experts * sum_e f_e * P_e`` over the local tokens), averaged over the
    data-parallel group for logging, scaled by ``moe_loss_coeff``."""
    if not moe_losses:
        return 0.0, 0.0
    lbl = torch.stack([m.float() for m in moe_losses]).mean()
    scaled = neox_args.moe_loss_coeff * lbl
    avg = scaled.detach().clone()
    if dist.is_available() and dist.is_initialized() and mpu.get_data_parallel_world_size() > 1:
        dist.all_reduce(avg, group=mpu.get_data_parallel_group())
        avg = avg / mpu.get_data_parallel_world_size()
    return scaled, avg


def _outputs(maybe_tuple):
    return maybe_tuple if isinstance(maybe_tuple, tuple) else (maybe_tuple, [])


def forward_step(data_iterator, model, neox_args, timers, return_logits=False, is_train=False, reference_model=None):
    """Forward one micro-batch and return ``(loss, metrics)`` (``(loss, logits, metrics)`` with
    ``return_logits``).  Under pipeline parallelism this is an ``eval_batch``."""
    if neox_args.is_pipe_parallel:
        return model.eval_batch(data_iterator, return_logits=return_logits)
    if timers is not None:
        timers("batch generator").start()
    with _nvtx(neox_args, "Get batch"):
        batch = get_batch(neox_args, data_iterator)
    if timers is not None:
        timers("batch generator").stop()
    impl = neox_args.train_impl
    tokens, labels, loss_mask, attention_mask, position_ids = batch[:5]
    metrics = {}
    fwd_in = (tokens, position_ids, attention_mask)
    with _nvtx(neox_args, "Forward pass"):
        if impl == "normal":
            outputs, moe_losses = _outputs(model(fwd_in, neox_args=neox_args))
            if is_train and neox_args.curriculum_learning and neox_args.curriculum_seqlen < neox_args.seq_length:
                loss_mask = loss_mask[:, : neox_args.curriculum_seqlen].contiguous()
                labels = labels[:, : neox_args.curriculum_seqlen].contiguous()
            loss = cross_entropy(outputs, (labels, loss_mask), _fp16=neox_args.fp16_lm_cross_entropy)
            if neox_args.moe_num_experts > 1:
                if neox_args.moe_type == "deepspeed":
                    # reference semantics: the summed per-layer losses enter as a detached constant
                    loss = loss + neox_args.moe_loss_coeff * sum(float(m) for m in moe_losses)
                else:
                    moe_loss, moe_avg = mb_moe_loss_func(neox_args, moe_losses)
                    metrics["moe_loss"] = moe_avg
                    loss = loss + moe_loss
        elif impl == "rm":
            outputs, _ = _outputs(model(fwd_in, neox_args=neox_args))
            loss, metrics = OBJ.reward_model_loss(outputs, loss_mask, neox_args.z_loss)
        elif impl == "dpo":
            ref_logp = batch[5]
            ref_out = None
            if not neox_args.dpo_reference_free and ref_logp is None:
                with torch.no_grad():
                    ref_out, _ = _outputs(reference_model(fwd_in, neox_args=neox_args))
            outputs, _ = _outputs(model(fwd_in, neox_args=neox_args))
            loss, metrics = OBJ.dpo_loss(outputs, labels, loss_mask, neox_args.dpo_beta, ref_logits=ref_out,
                                         ref_logp=ref_logp, reference_free=neox_args.dpo_reference_free,
                                         fp32=neox_args.dpo_fp32)
        elif impl == "kto":
            rewards, ref_logp = batch[5], batch[6]
            ref_out = None
            if ref_logp is None:
                with torch.no_grad():
                    ref_out, _ = _outputs(reference_model(fwd_in, neox_args=neox_args))
            outputs, _ = _outputs(model(fwd_in, neox_args=neox_args))
            loss, metrics = OBJ.kto_loss(outputs, labels, loss_mask, rewards, neox_args.kto_beta,
                                         neox_args.kto_desirable_weight, neox_args.kto_undesirable_weight,
                                         ref_logits=ref_out, ref_logp=ref_logp, fp32=neox_args.kto_fp32)
        elif impl == "reinforce":
            rewards, raw_rewards = batch[5], batch[6]
            ref_out = None
            if reference_model is not None:
                with torch.no_grad():
                    ref_out, _ = _outputs(reference_model(fwd_in, neox_args=neox_args))
            outputs, _ = _outputs(model(fwd_in, neox_args=neox_args))
            loss, metrics = OBJ.reinforce_loss(outputs, labels, loss_mask, rewards, raw_rewards, neox_args.kl_impl,
                                               neox_args.kl_div_beta, ref_logits=ref_out,
                                               fp32=neox_args.fp32_reinforce)
        else:
            raise ValueError(f"unknown train_impl {impl}")
    if return_logits:
        return loss, outputs, metrics
    return loss, metrics


# ------------------------------------------------------------------------------------ model / optimizer
def get_model(neox_args, use_cache=False, park_on_host=False):
    """Build the model on this rank (``megatron/training.py:947-1033``).  ``park_on_host``: see below."""
    print_rank_0("building GPT2 model ...")
    if neox_args.zero_stage in (2, 3):
        if neox_args.pipe_parallel_size == 1:
            print_rank_0("ZeRO stage 2/3 and the PipelineModule are incompatible, please set 'pipe_parallel_size' to 0 instead")
            sys.exit(1)
        if neox_args.pipe_parallel_size > 1:
            print_rank_0("ZeRO stage 2/3 and pipeline paralleism are not supported simultaneously")
            sys.exit(1)
        # (the reference also refuses model parallelism here, ``megatron/training.py:968-973``; this engine's
        # gradient partitioning works per data-parallel group and composes with tensor / sequence parallelism)
    # stage 3 with parameter offload: every layer is parked in host memory as soon as it has been built and
    # initialised, and the optimizer later brings it to the device one bucket at a time, keeping only this rank's
    # shard -- the model never exists in full on the device (the role of ``deepspeed.zero.Init(remote_device="cpu")``,
    # ``megatron/training.py:958-977``)
    through_host = contextlib.nullcontext()
    if park_on_host:
        from .engine.pipe_module import built_through
        through_host = built_through(lambda layer: layer.to("cpu"))
    with through_host:
        model = GPT2ModelPipe(neox_args=neox_args, num_tokentypes=0, parallel_output=neox_args.train_impl != "rm",
                              topology=mpu.get_topology(), use_cache=use_cache)
    if neox_args.soft_prompt_tuning is not None and neox_args.soft_prompt_tuning.get("enabled", False):
        spt = neox_args.soft_prompt_tuning
        soft = SoftEmbedding(neox_args, wte=getattr(model, "0").word_embeddings if hasattr(model, "0")
                             else model.tied_modules["embed"].word_embeddings,
                             n_tokens=spt.get("num_tokens", 10), init_string=spt.get("init_string", ""),
                             init_range=spt.get("init_range", 0.5))
        model.insert_layers(layers=soft, idx=1)
        for name, p in model.named_parameters():
            if "soft_embedding" not in name:
                p.requires_grad = False
    if not neox_args.is_pipe_parallel:
        model = model.to_sequential()
    if neox_args.use_mup:
        from .mup_support import apply_mup
        apply_mup(model, neox_args)
    return model


def _train_device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def optimizer_offload(neox_args) -> bool:
    """Whether the fp32 masters and optimizer states live in host memory: a host optimizer type, or the ZeRO
    configuration asks for it (``cpu_offload: true``, or ``offload_optimizer: {device: cpu}``)."""
    z = neox_args.zero_optimization or {}
    off = z.get("offload_optimizer") or {}
    return bool(z.get("cpu_offload")) or str(off.get("device", "none")).lower() == "cpu" or \
        neox_args.optimizer_type.lower() in ("cpu_adam", "cpu_torch_adam")


def param_offload(neox_args) -> bool:
    """ZeRO stage 3 with the persistent parameter shards in host memory (``offload_param: {device: cpu}``)."""
    z = neox_args.zero_optimization or {}
    off = z.get("offload_param") or {}
    return neox_args.zero_stage == 3 and str(off.get("device", "none")).lower() == "cpu"


def _numeric(v):
    """YAML 1.1 reads ``1e-8`` (no dot) as a string: give optimizer hyper-parameters written that way their value."""
    if isinstance(v, str):
        try:
            return float(v)
        except ValueError:
            return v
    if isinstance(v, (list, tuple)):
        return type(v)(_numeric(x) for x in v)
    return v


def _inner_optimizer(neox_args):
    """(class, kwargs) of the element-wise optimizer that updates the flat fp32 shards."""
    name = neox_args.optimizer_type.lower()
    params = {k: _numeric(v) for k, v in dict(neox_args.optimizer.get("params", {})).items()}
    params.pop("freeze_step", None) if name != "onebitadam" else None
    if name in ("adam", "cpu_adam", "cpu_torch_adam", "onebitadam"):
        if name == "cpu_torch_adam":
            params.pop("cuda_aware", None)
            return torch.optim.Adam, dict(weight_decay=neox_args.weight_decay, **params)
        if name == "cpu_adam" or (name == "adam" and optimizer_offload(neox_args)):
            from .optim.cpu_adam import CPUAdam
            return CPUAdam, dict(weight_decay=neox_args.weight_decay, **params)
        if name == "onebitadam":
            from .optim.onebit_adam import OneBitAdam
            return OneBitAdam, dict(weight_decay=neox_args.weight_decay, comm_group=mpu.get_data_parallel_group(),
                                    **params)
        params.pop("cuda_aware", None)
        params.pop("momentum", None)
        if neox_args.use_bnb_optimizer:
            from .optim.adam8bit import Adam8bit
            return Adam8bit, dict(weight_decay=neox_args.weight_decay, **params)
        from .optim.fused_adam import FusedAdam
        return FusedAdam, dict(weight_decay=neox_args.weight_decay, **params)
    if name == "sm3":
        from .optim.sm3 import SM3
        return SM3, params
    if name == "madgrad_wd":
        from .optim.madgrad import madgrad_wd
        return madgrad_wd, dict(weight_decay=neox_args.weight_decay, **params)
    if name == "lion":
        from .optim.lion import Lion
        return Lion, dict(weight_decay=neox_args.weight_decay, **params)
    if name == "sgd":
        return torch.optim.SGD, dict(weight_decay=neox_args.weight_decay, **params)
    raise ValueError(f"Optimizer type {neox_args.optimizer_type} not recognized")


def get_optimizer(model, neox_args, dummy=False):
    """Parameter groups -> flat sharded mixed-precision optimizer.  Returns ``(optimizer, param_groups)``."""
    if neox_args.no_load_optim or neox_args.optimizer is None:
        if neox_args.optimizer is None and not neox_args.no_load_optim:
            print_rank_0("ERROR: Optimizer is None. Either set the optimizer dict in your config (if training) or "
                         "set no_load_optim in your config (if inference)")
            sys.exit(1)
        return None, None
    groups = get_params_for_weight_decay_optimization(model, neox_args)
    groups = [dict(g) for g in (groups if isinstance(groups, (list, tuple)) else [groups])]
    print_rank_0(f'Configuring Optimizer type: {neox_args.optimizer_type} with params: {neox_args.optimizer["params"]}')
    seen = set()
    for g in groups:
        uniq = []
        for p in g["params"]:
            if not hasattr(p, "model_parallel"):
                p.model_parallel = False
            if p.requires_grad and id(p) not in seen:
                seen.add(id(p))
                uniq.append(p)
        g["params"] = uniq
        g.pop("name", None)
    assert not neox_args.use_mup or neox_args.optimizer_type.lower() in ("adam", "sgd"), \
        f"If use_mup == True, you must specify either the adam or sgd optimizers. You passed: {neox_args.optimizer_type.lower()}"
    inner_cls, inner_kw = _inner_optimizer(neox_args)
    flat_ok = neox_args.optimizer_type.lower() != "sm3"
    if not flat_ok:
        # SM3 keeps per-row/column accumulators and needs the real parameter shapes: plain optimizer
        opt = inner_cls([{"params": g["params"], **{k: v for k, v in g.items() if k != "params"}} for g in groups
                         if g["params"]], **inner_kw)
        from .engine.plain_optimizer import PlainOptimizer
        return PlainOptimizer(opt, clip_grad=neox_args.gradient_clipping), groups
    fp16_cfg = dict(neox_args.fp16 or {})
    # tags (late_grad_sync) must be in place before the optimizer lays out its buckets
    mark_norms_for_sequence_parallel_grad_sync(model, neox_args)
    optimizer = FlatMixedPrecisionOptimizer(groups, inner_cls, inner_kw, neox_args.params_dtype,
                                            zero_stage=neox_args.zero_stage if isinstance(neox_args.zero_stage, int) else 0,
                                            clip_grad=neox_args.gradient_clipping, fp16_cfg=fp16_cfg,
                                            overlap_comm=bool((neox_args.zero_optimization or {}).get("overlap_comm", False)),
                                            reduce_bucket_size=neox_args.zero_reduce_bucket_size,
                                            offload_optimizer=optimizer_offload(neox_args),
                                            partition_params_at_build=param_offload(neox_args),
                                            offload_param=param_offload(neox_args),
                                            device=_train_device() if param_offload(neox_args) else None)
    if param_offload(neox_args):
        model.to(_train_device())      # buffers and parameters outside the optimizer follow; released ones are there
    if getattr(optimizer, "overlap_comm", False):
        # each layer waits only for the all-gather of its own parameters
        optimizer.install_param_wait_hooks(model)
    if optimizer.zero_stage >= 3:
        optimizer.enable_param_partitioning(model, offload_param=param_offload(neox_args))
    return optimizer, groups


def get_learning_rate_scheduler(optimizer, neox_args):
    if optimizer is None:
        return None
    if neox_args.lr_decay_iters is not None:
        num_iters = neox_args.lr_decay_iters
    elif neox_args.lr_decay_fraction is not None:
        num_iters = math.floor(neox_args.train_iters * neox_args.lr_decay_fraction)
    else:
        num_iters = neox_args.train_iters
    num_iters = max(1, num_iters or 1)
    return AnnealingLR(optimizer, start_lr=neox_args.lr, warmup_iter=neox_args.warmup * num_iters,
                       total_iters=num_iters, decay_style=neox_args.lr_decay_style, last_iter=0,
                       min_lr=neox_args.min_lr, use_checkpoint_lr_scheduler=neox_args.use_checkpoint_lr_scheduler,
                       override_lr_scheduler=neox_args.override_lr_scheduler, use_mup=neox_args.use_mup)


def dump_engine_state(engine, neox_args):
    """``dump_state``: what the engine was built with, printed once by rank 0 after initialisation."""
    opt = engine.optimizer
    rows = {
        "engine": type(engine).__name__,
        "world (data x pipe x model)": f"{mpu.get_data_parallel_world_size()} x {mpu.get_pipe_parallel_world_size()} "
                                       f"x {mpu.get_model_parallel_world_size()}",
        "train_batch_size": neox_args.train_batch_size,
        "train_micro_batch_size_per_gpu": neox_args.train_micro_batch_size_per_gpu,
        "gradient_accumulation_steps": neox_args.gradient_accumulation_steps,
        "precision": neox_args.precision,
        "gradient_clipping": neox_args.gradient_clipping,
        "total_params": getattr(engine, "total_params", None),
        "optimizer": type(getattr(opt, "optimizer", opt)).__name__ if opt is not None else None,
        "zero_stage": getattr(opt, "zero_stage", None),
        "overlap_comm": getattr(opt, "overlap_comm", None),
        "offload_optimizer": getattr(opt, "offload_optimizer", None),
        "buckets": len(getattr(opt, "buckets", []) or []),
        "bucket elements (largest)": max((b.padded for b in getattr(opt, "buckets", []) or []), default=0),
        "loss_scale": opt.cur_scale if opt is not None and hasattr(opt, "cur_scale") else None,
        "lr_scheduler": type(engine.lr_scheduler).__name__ if engine.lr_scheduler is not None else None,
        "wall_clock_breakdown": engine.wall_clock_breakdown(),
        "steps_per_print": engine.steps_per_print(),
    }
    print_rank_0("engine state:")
    for k, v in rows.items():
        print_rank_0(f"  {k} {'.' * max(1, 34 - len(k))} {v}")
    return rows


def setup_model_and_optimizer(neox_args, use_cache=False, iteration=None):
    """Model, optimizer, scheduler, engine and (optionally) checkpoint restore.
    Returns ``(engine, optimizer, lr_scheduler, reference_model)``."""
    if neox_args.memory_profiling and torch.cuda.is_available():
        torch.cuda.memory._record_memory_history(True, trace_alloc_max_entries=100000, trace_alloc_record_context=True)
    will_train = neox_args.optimizer is not None and not neox_args.no_load_optim
    model = get_model(neox_args=neox_args, use_cache=use_cache, park_on_host=param_offload(neox_args) and will_train)
    needs_reference = (neox_args.train_impl == "dpo" and neox_args.precompute_model_name is None
                       and not neox_args.dpo_reference_free) or \
                      (neox_args.train_impl == "kto" and neox_args.precompute_model_name is None)
    reference_model = get_model(neox_args=neox_args, use_cache=use_cache) if needs_reference else None
    optimizer, param_groups = get_optimizer(model=model, neox_args=neox_args)
    lr_scheduler = get_learning_rate_scheduler(optimizer=optimizer, neox_args=neox_args)
    sp_params = mark_norms_for_sequence_parallel_grad_sync(model, neox_args)
    engine_cls = PipelineEngine if neox_args.is_pipe_parallel else NeoXEngine
    engine = engine_cls(model, optimizer, lr_scheduler, neox_args, sp_sync_params=sp_params)
    if reference_model is not None:
        reference_model = NeoXEngine(reference_model, None, None, neox_args)
    engine.total_params = get_total_params(model)
    print_rank_0(f' > total params: {"{:,}".format(engine.total_params)}')
    if neox_args.is_pipe_parallel:
        engine.set_has_attention_mask(True)
        curr = None
        if neox_args.curriculum_learning:
            from .engine.curriculum import CurriculumScheduler
            curr = CurriculumScheduler(neox_args.curriculum_learning)
            if iteration is not None and iteration > 0:
                curr.update_difficulty(iteration)
        engine.set_batch_fn(partial(get_batch_pipe, neox_args=neox_args, curr_scheduler=curr))
        if curr is not None:
            engine.set_curriculum_scheduler(curr)
    if neox_args.dump_state:
        dump_engine_state(engine, neox_args)
    if neox_args.load is not None:
        neox_args.iteration = load_checkpoint(neox_args=neox_args, model=engine, optimizer=optimizer,
                                              lr_scheduler=lr_scheduler, iteration=iteration)
        if reference_model is not None:
            load_checkpoint(neox_args=neox_args, model=reference_model, optimizer=None, lr_scheduler=None,
                            iteration=iteration)
        print_rank_0(f"Loading checkpoint and starting from iteration {neox_args.iteration}")
    else:
        neox_args.iteration = 0
    if lr_scheduler is not None and neox_args.iteration:
        lr_scheduler.optimizer = engine.optimizer
    return engine, optimizer, lr_scheduler, reference_model


# ------------------------------------------------------------------------------------ steps
def backward_step(neox_args, timers, optimizer, model, loss):
    if timers is not None:
        timers("backward-backward").start()
    model.backward(loss)
    if timers is not None:
        timers("backward-backward").stop()


def train_step(neox_args, timers, data_iterator, model, optimizer, lr_scheduler, reference_model=None):
    """One optimizer step = ``gradient_accumulation_steps`` micro-batches."""
    if neox_args.is_pipe_parallel:
        reduced_loss = train_step_pipe(neox_args, timers, model, data_iterator)
        reduce_metrics = reduced_loss
    else:
        losses, metric_dicts = [], {}
        for _ in range(neox_args.gradient_accumulation_steps):
            timers("forward").start()
            loss, metrics = forward_step(neox_args=neox_args, timers=timers, data_iterator=data_iterator, model=model,
                                         is_train=True, reference_model=reference_model)
            timers("forward").stop()
            losses.append(loss)
            for k, v in metrics.items():
                metric_dicts.setdefault(k, []).append(v)
            timers("backward").start()
            with _nvtx(neox_args, "Backward pass"):
                backward_step(neox_args, timers, optimizer, model, loss)
            timers("backward").stop()
            timers("optimizer").start()
            with _nvtx(neox_args, "Optimizer step"):
                model.step()
            timers("optimizer").stop()
        reduce_metrics = {k: reduce_losses([torch.as_tensor(x, device=losses[0].device).float() for x in v]).mean()
                          for k, v in metric_dicts.items()}
        reduce_metrics["lm_loss"] = reduce_losses(losses).mean()
    skipped_iter = 1 if (neox_args.precision == "fp16" and model.optimizer is not None
                         and getattr(model.optimizer, "overflow", False)) else 0
    collect_loss_for_unit_test(reduce_metrics["lm_loss"])
    return reduce_metrics, skipped_iter


def train_step_pipe(neox_args, timers, model, data_iterator):
    loss = model.train_batch(data_iter=data_iterator)
    return {"lm_loss": loss}


def collect_loss_for_unit_test(lm_loss):
    """Hook patched by tests to observe the per-step loss."""
    pass


class _TrialMetric:
    """Throughput of an autotuning trial: wall-clock (device-synchronised) between ``autotuning.start_profile_step``
    and ``end_profile_step``, written by rank 0 to ``autotuning_metric_path`` (read back by ``autotuning.Autotuner``)."""

    def __init__(self, neox_args):
        block = neox_args.autotuning or {}
        self.args = neox_args
        self.start = int(block.get("start_profile_step", 3))
        self.end = int(block.get("end_profile_step", 5))
        self.t0 = None

    @staticmethod
    def _now():
        import time
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        return time.perf_counter()

    def before_step(self, iteration):
        if iteration == self.start:
            self.t0 = self._now()
        elif iteration == self.end and self.t0 is not None:
            dt = (self._now() - self.t0) / max(self.end - self.start, 1)
            if (not dist.is_initialized()) or dist.get_rank() == 0:
                import json
                with open(self.args.autotuning_metric_path, "w") as fh:
                    json.dump({"latency": dt, "throughput": self.args.train_batch_size / dt,
                               "tokens_per_sec": self.args.train_batch_size * self.args.seq_length / dt}, fh)
            self.t0 = None


def train(neox_args, timers, model, optimizer, lr_scheduler, train_data_iterator, valid_data_iterator,
          reference_model=None):
    model.train()
    total_loss_dict = {}
    iteration = neox_args.iteration
    timers("interval time").start()
    report_memory_flag = True
    noise_scale_logger = get_noise_scale_logger(neox_args)
    if noise_scale_logger is not None:
        noise_scale_logger = noise_scale_logger(model)
    overflow_monitor = OverflowMonitor(optimizer)
    ds_cfg = neox_args.deepspeed_config
    comms = comms_logger.configure(neox_args.comms_logger or ds_cfg.get("comms_logger"))
    from .logging import configure_csv_monitor
    configure_csv_monitor(neox_args.csv_monitor or ds_cfg.get("csv_monitor"))
    flops_prof = FlopsProfiler.from_config(getattr(model, "module", model),
                                           neox_args.flops_profiler or ds_cfg.get("flops_profiler"))
    prof = None
    if neox_args.profile and torch.cuda.is_available():
        sched = torch.profiler.schedule(wait=neox_args.profile_step_start, warmup=1,
                                        active=neox_args.profile_step_stop - neox_args.profile_step_start)
        prof = torch.profiler.profile(schedule=sched,
                                      on_trace_ready=torch.profiler.tensorboard_trace_handler(neox_args.tensorboard_dir or "./tb"),
                                      record_shapes=True, profile_memory=True, with_flops=True, with_modules=True,
                                      with_stack=True)
        prof.start()
    tune = _TrialMetric(neox_args) if neox_args.autotuning_metric_path else None
    while iteration < neox_args.train_iters:
        if tune is not None:
            tune.before_step(iteration)
        if prof is not None:
            prof.step()
        if neox_args.profile and iteration == neox_args.profile_step_start and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStart()
        profiling_flops = flops_prof.enabled and iteration + 1 == flops_prof.profile_step
        if profiling_flops:
            flops_prof.start_profile()
        loss_dict, skipped_iter = train_step(neox_args=neox_args, timers=timers, data_iterator=train_data_iterator,
                                             model=model, optimizer=optimizer, lr_scheduler=lr_scheduler,
                                             reference_model=reference_model)
        if profiling_flops:
            flops_prof.stop_profile()
            print_rank_0(flops_prof.report(batch_size=neox_args.train_batch_size // max(mpu.get_data_parallel_world_size(), 1)))
        if comms.enabled and (iteration + 1) % neox_args.log_interval == 0:
            comms.log_summary()
        if neox_args.profile and iteration == neox_args.profile_step_stop and torch.cuda.is_available():
            torch.cuda.cudart().cudaProfilerStop()
            if prof is not None:
                prof.stop()
                prof = None
        iteration += 1
        neox_args.iteration = iteration
        if neox_args.precision == "fp16":
            overflow_monitor.check(skipped_iter)
        if noise_scale_logger is not None:
            noise_scale_logger.update()
        lr = optimizer.param_groups[0].get("lr", 0) if optimizer is not None else 0
        report_memory_flag = training_log(neox_args=neox_args, timers=timers, loss_dict=loss_dict,
                                          total_loss_dict=total_loss_dict, learning_rate=lr, iteration=iteration,
                                          loss_scale=optimizer.cur_scale if (neox_args.precision == "fp16" and optimizer is not None) else None,
                                          report_memory_flag=report_memory_flag, skipped_iter=skipped_iter,
                                          model=model, optimizer=optimizer, noise_scale_logger=noise_scale_logger)
        if neox_args.save and is_save_iter(neox_args, iteration):
            save_checkpoint(neox_args=neox_args, iteration=iteration, model=model, optimizer=optimizer,
                            lr_scheduler=lr_scheduler)
        if neox_args.eval_interval and iteration % neox_args.eval_interval == 0 and neox_args.do_valid:
            evaluate_and_print_results(neox_args=neox_args, prefix=f"iteration {iteration}", forward_step_func=forward_step,
                                       data_iterator=valid_data_iterator, model=model, iteration=iteration,
                                       verbose=False, timers=timers, reference_model=reference_model)
        if neox_args.exit_interval and iteration % neox_args.exit_interval == 0:
            if dist.is_available() and dist.is_initialized():
                dist.barrier()
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
            print(f"rank: {rank} | exiting the program at iteration {iteration}", flush=True)
            sys.exit()
    return iteration


def evaluate(neox_args, forward_step_fn, data_iterator, model, verbose=False, timers=None, reference_model=None):
    """Average losses over ``eval_iters`` iterations (x ``gradient_accumulation_steps`` micro-batches when
    not pipelined, so that the number of evaluated samples matches the pipeline path)."""
    model.eval()
    losses, metric_dicts = [], {}
    if neox_args.char_level_ppl:
        data_iterator = CharCounter(data_iterator, neox_args.tokenizer)
    with torch.no_grad():
        iteration = 0
        while iteration < neox_args.eval_iters:
            iteration += 1
            if verbose and iteration % neox_args.log_interval == 0:
                print_rank_0(f"Evaluating iter {iteration}/{neox_args.eval_iters}")
            for _ in range(1 if neox_args.is_pipe_parallel else neox_args.gradient_accumulation_steps):
                out = forward_step_fn(model=model, data_iterator=data_iterator, neox_args=neox_args, timers=timers,
                                      reference_model=reference_model)
                loss, metrics = out if isinstance(out, tuple) else (out, {})
                losses.append(loss)
                for k, v in metrics.items():
                    metric_dicts.setdefault(k, []).append(v)
    eval_results = {"lm_loss": reduce_losses(losses).mean().item()}
    for k, v in metric_dicts.items():
        eval_results[k] = reduce_losses([torch.as_tensor(x).float().to(losses[0].device) for x in v]).mean().item()
    eval_results["lm_loss_ppl"] = math.exp(min(20, eval_results["lm_loss"]))
    if neox_args.char_level_ppl:
        tpc = data_iterator.tokens_per_char()
        eval_results["lm_loss_char_lvl_ppl"] = math.exp(eval_results["lm_loss"] * tpc)
    if neox_args.eval_tasks:
        from .eval_tasks import run_eval_harness
        eval_results.update(run_eval_harness(model, forward_step_fn, neox_args, eval_tasks=neox_args.eval_tasks)
                            .get("results", {}))
    model.train()
    return eval_results


def evaluate_and_print_results(neox_args, prefix, forward_step_func, data_iterator, model, iteration, verbose=False,
                               timers=None, chart_name="validation", reference_model=None):
    total_loss_dict = evaluate(neox_args=neox_args, forward_step_fn=forward_step_func, data_iterator=data_iterator,
                               model=model, verbose=verbose, timers=timers, reference_model=reference_model)
    string = f" {chart_name} results at {prefix} | "
    for k, v in total_loss_dict.items():
        if isinstance(v, dict):
            if neox_args.eval_tasks and "results" in v:
                v = v["results"]
            for k2, v2 in v.items():
                k3 = "_".join([k, k2])
                string += f"{k3} value: {v2:.6E} | " if isinstance(v2, (int, float)) else f"{k3} value: {v2} | "
                if isinstance(v2, (int, float)):
                    tb_wandb_log(f"{chart_name}/{k3}", v2, iteration, use_wandb=neox_args.use_wandb,
                                 tensorboard_writer=neox_args.tensorboard_writer, comet_experiment=neox_args.comet_experiment)
        else:
            string += f"{k} value: {v:.6E} | "
            tb_wandb_log(f"{chart_name}/{k}", v, iteration, use_wandb=neox_args.use_wandb,
                         tensorboard_writer=neox_args.tensorboard_writer, comet_experiment=neox_args.comet_experiment)
    length = len(string) + 1
    print_rank_0("-" * length)
    print_rank_0(string)
    print_rank_0("-" * length)
    return total_loss_dict


# ------------------------------------------------------------------------------------ entry
def pretrain(neox_args):
    """Initialise everything, train, validate, test, save."""
    from .utils.wandb import init_wandb
    init_wandb(neox_args=neox_args)
    timers = Timers(use_wandb=neox_args.use_wandb, tensorboard_writer=neox_args.tensorboard_writer,
                    comet_experiment=neox_args.comet_experiment)
    initialize_megatron(neox_args=neox_args)
    timers("train/valid/test data loaders").start()
    train_dl, valid_dl, test_dl = build_train_valid_test_data_loaders(neox_args=neox_args)
    timers("train/valid/test data loaders").stop()
    if neox_args.train_iters is None and neox_args.train_epochs is not None:
        update_iterations(neox_args, {"train": train_dl})
    timers("model and optimizer").start()
    model, optimizer, lr_scheduler, reference_model = setup_model_and_optimizer(neox_args=neox_args, use_cache=False,
                                                                               iteration=neox_args.iteration)
    timers("model and optimizer").stop()
    if neox_args.serve_model_weights:
        from .weight_server import start_server
        start_server(model)
        if dist.is_available() and dist.is_initialized():
            dist.barrier()
    train_it, valid_it, test_it = shift_and_wrap_data_loaders(neox_args, train_dl, valid_dl, test_dl)
    if neox_args.use_mup and neox_args.coord_check:
        # muP coordinate check: a diagnostic run that replaces training (reference: training.py:273-275)
        from .mup_support import mup_coord_check
        mup_coord_check(neox_args, timers, train_it)
        print_rank_0("coordinate check written to coord_check_up.* / coord_check_sp.*; exiting")
        sys.exit(0)
    print_rank_0("done with setups ...")
    timers.log(["train/valid/test data loaders", "model and optimizer"])
    print_rank_0("training ...")
    iteration = neox_args.iteration
    if neox_args.save and neox_args.extra_save_iters and 0 in neox_args.extra_save_iters and iteration == 0:
        save_checkpoint(neox_args=neox_args, iteration=iteration, model=model, optimizer=optimizer,
                        lr_scheduler=lr_scheduler)
    if neox_args.do_train and neox_args.train_iters > 0:
        iteration = train(neox_args=neox_args, timers=timers, model=model, optimizer=optimizer,
                          lr_scheduler=lr_scheduler, train_data_iterator=train_it, valid_data_iterator=valid_it,
                          reference_model=reference_model)
    if neox_args.do_valid:
        evaluate_and_print_results(neox_args=neox_args, prefix="the end of training for val data",
                                   forward_step_func=forward_step, data_iterator=valid_it, model=model,
                                   iteration=iteration, verbose=False, timers=timers, reference_model=reference_model)
    if neox_args.save and iteration != 0 and not is_save_iter(neox_args, iteration):
        save_checkpoint(neox_args=neox_args, iteration=iteration, model=model, optimizer=optimizer,
                        lr_scheduler=lr_scheduler)
    if neox_args.do_test:
        evaluate_and_print_results(neox_args=neox_args, prefix="the end of training for test data",
                                   forward_step_func=forward_step, data_iterator=test_it, model=model,
                                   iteration=iteration, verbose=True, timers=timers, chart_name="test",
                                   reference_model=reference_model)
    if neox_args.memory_profiling and torch.cuda.is_available() and (neox_args.rank or 0) == 0:
        import pickle
        snap = torch.cuda.memory._snapshot()
        with open((neox_args.memory_profiling_path or ".") + "/mem_snapshot.pickle", "wb") as fh:
            pickle.dump(snap, fh)
    return model
