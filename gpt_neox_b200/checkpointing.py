"""Checkpoint save / load with the on-disk layout GPT-NeoX tooling expects.

Layout written under ``<save>/`` (what DeepSpeed's engine writes for the reference,
``megatron/checkpointing.py:181-223`` + ``tools/ckpts/convert_neox_to_hf.py:165-205``)::

    latest                                       text file holding the newest tag
    global_step{N}/
        mp_rank_{tp:02d}_model_states.pt         sequential model: {"module": {"sequential.{idx}.{name}": tensor},
                                                 "optimizer": None, "lr_scheduler", "dp_world_size", "mp_world_size",
                                                 "global_steps", "global_samples", "skipped_steps", "iteration", + client state}
        layer_{idx:02d}-model_{tp:02d}-model_states.pt   pipeline model: one bare state dict per layer owned by a stage
        zero_pp_rank_{dp}_mp_rank_{tp:02d}_optim_states.pt   one optimizer shard per data-parallel rank
                                                 (prefix ``bf16_`` for bf16 runs).  Pipeline runs keep the weights
                                                 only in the per-layer files above; their ``mp_rank_*`` files hold
                                                 the engine counters and client state.
        configs/*.yml                            verbatim copies of the launch configs

Client state: ``iteration``, a subset of args for consistency checks, five RNG states, optional
validation logits.  ``keep_last_n_checkpoints`` garbage-collects old tags; ``s3_path`` mirrors the
tag directory to S3 when boto3 is importable.
"""
from __future__ import annotations

import json
import os
import random
import re
import shutil
import sys

import numpy as np
import torch
import torch.distributed as dist

from .parallel import mpu
from .parallel.rng import get_cuda_rng_tracker
from .utils import natural_sort, print_rank_0

_CHECK_ARGS = ("num_layers", "hidden_size", "num_attention_heads", "max_position_embeddings",
               "make_vocab_size_divisible_by", "padded_vocab_size", "tokenizer_type", "model_parallel_size")


def _dist_on():
    return dist.is_available() and dist.is_initialized()


def _barrier():
    if _dist_on():
        dist.barrier()


def _rank():
    return dist.get_rank() if _dist_on() else 0


def get_checkpoint_tag(iteration: int) -> str:
    return f"global_step{iteration}"


def check_checkpoint_args(neox_args, checkpoint_args):
    assert isinstance(checkpoint_args, dict), "args stored in checkpoint is a dict"
    for name, saved in checkpoint_args.items():
        cur = getattr(neox_args, name)
        assert saved == cur, f"{name} value from checkpoint ({saved}) is not equal to the currently set argument value ({cur})."


def do_forward_pass(neox_args, model, inference=False):
    """Deterministic probe: logits of ``arange(seq_length)`` for the first batch row."""
    was_training = model.module.training
    model.module.eval()
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    ctx = torch.arange(neox_args.seq_length + 1).repeat((neox_args.train_micro_batch_size_per_gpu, 1)).to(dev)
    ctx = ctx % neox_args.padded_vocab_size
    with torch.no_grad():
        if neox_args.is_pipe_parallel:
            _, logits = model.eval_batch(data_iter=iter([{"text": ctx}]), return_logits=True, num_micro_batches=1)
        else:
            tokens = ctx[:, :neox_args.seq_length].contiguous()
            pos = torch.arange(neox_args.seq_length, device=dev).unsqueeze(0).expand_as(tokens)
            out = model((tokens, pos, None))
            logits = out[0] if isinstance(out, tuple) else out
    if was_training:
        model.module.train()
    return logits.detach().float().cpu()[0] if logits is not None else None


def check_forward_pass(neox_args, model, checkpoint_logits, inference):
    logits = do_forward_pass(neox_args=neox_args, model=model, inference=inference)
    if logits is not None and checkpoint_logits is not None:
        if not (logits == checkpoint_logits).all().item():
            if mpu.get_data_parallel_rank() == 0:
                print(" > WARNING: validate_checkpoint_forward() forward after load of checkpoint does not yield "
                      "exactly same result")
            assert torch.isclose(logits, checkpoint_logits).all().item(), \
                "validate_checkpoint_forward() forward after load of checkpoint does not yield a close result"


# ------------------------------------------------------------------------------------ engine-level writer
def _optim_file(save_dir, tag, bf16, dp_rank=None):
    prefix = "bf16_" if bf16 else ""
    dp_rank = mpu.get_data_parallel_rank() if dp_rank is None else dp_rank
    return os.path.join(save_dir, tag, f"{prefix}zero_pp_rank_{dp_rank}_mp_rank_{_mp_file_rank():02d}_optim_states.pt")


def _expert_params(module):
    """``{name: parameter}`` of the parameters that differ between expert-parallel ranks."""
    return {n: p for n, p in module.named_parameters() if getattr(p, "expert_parallel", False)}


def _expert_file(d):
    """Experts are split over the expert-parallel ranks of a data-parallel group, so the shared model files (written
    by data-parallel rank 0) hold only that rank's experts; every expert-parallel rank keeps its own in this file."""
    return os.path.join(d, f"expert_ep_rank_{mpu.get_expert_parallel_rank():02d}_mp_rank_{_mp_file_rank():02d}"
                           "_model_states.pt")


def _per_rank_optimizer_state(engine) -> bool:
    """Whether every data-parallel rank holds optimizer state of its own: ZeRO shards, experts of its own, or an
    optimizer that says so (the error-feedback buffers of compressed communication)."""
    inner = getattr(engine.optimizer, "optimizer", engine.optimizer)
    return getattr(engine.optimizer, "zero_stage", 0) >= 1 or mpu.get_expert_parallel_world_size() > 1 or \
        bool(getattr(inner, "rank_local_state", False))


def _atomic_save(obj, path):
    """Write through a temporary name and rename: a run that is killed while writing never leaves a truncated file
    under the final name."""
    tmp = f"{path}.tmp.{os.getpid()}"
    try:
        torch.save(obj, tmp)
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


def _read(path):
    """``torch.load`` with an error that names the damaged file."""
    try:
        return torch.load(path, map_location="cpu", weights_only=False)
    except Exception as exc:      # truncated zip, pickle error, ...
        raise CheckpointDamaged(f"checkpoint file {path} cannot be read ({type(exc).__name__}: {exc}); "
                                "it is truncated or corrupt") from exc


class CheckpointDamaged(RuntimeError):
    pass


COMPLETE_MARKER = ".complete"


def complete_tags(load_dir):
    """Tags under ``load_dir`` whose save ran to the end (newest first)."""
    if not os.path.isdir(load_dir):
        return []
    tags = [t for t in os.listdir(load_dir)
            if t.startswith("global_step") and os.path.isfile(os.path.join(load_dir, t, COMPLETE_MARKER))]
    return sorted(tags, key=lambda t: int(re.sub(r"\D", "", t) or 0), reverse=True)


def _mp_file_rank():
    """File index over the model-parallel grid: tp rank for sequential models, ``stage * tp + tp_rank``
    when the pipeline holds several stages."""
    return mpu.get_pipe_parallel_rank() * mpu.get_model_parallel_world_size() + mpu.get_model_parallel_rank()


def _is_pipe_module(module):
    from .engine.pipe_module import PipelineModule
    return isinstance(module, PipelineModule)


def _params_resident(engine, write_back=False):
    """Under ZeRO stage 3 the module's parameters exist in full only inside this context."""
    import contextlib
    part = getattr(engine.optimizer, "param_partitioner", None) if engine.optimizer is not None else None
    return part.all_resident(write_back=write_back) if part is not None else contextlib.nullcontext()


def engine_save_checkpoint(engine, save_dir, tag, client_state):
    with _params_resident(engine):
        return _engine_save_checkpoint(engine, save_dir, tag, client_state)


def _engine_save_checkpoint(engine, save_dir, tag, client_state):
    tag = tag or get_checkpoint_tag(engine.global_steps)
    d = os.path.join(save_dir, tag)
    os.makedirs(d, exist_ok=True)
    _barrier()
    tp = mpu.get_model_parallel_rank()
    module = engine.module
    writer = mpu.get_data_parallel_rank() == 0
    # the parameter all-gather of the last step may still be in flight on the optimizer's side stream
    if hasattr(engine.optimizer, "wait_all_params"):
        engine.optimizer.wait_all_params()
    common = {
        "optimizer": None,
        "lr_scheduler": engine.lr_scheduler.state_dict() if engine.lr_scheduler is not None else None,
        "dp_world_size": mpu.get_data_parallel_world_size(),
        "mp_world_size": mpu.get_model_parallel_world_size(),
        "global_steps": engine.global_steps,
        "global_samples": engine.global_samples,
        "skipped_steps": engine.skipped_steps,
        "ds_version": "neox-b200",
    }
    common.update(client_state)
    if _is_pipe_module(module):
        if writer:
            for idx in module.local_layer_indices():
                layer = module.layer_module(idx)
                if layer is None or not any(True for _ in layer.state_dict()):
                    continue
                _atomic_save({k: v.detach().cpu() for k, v in layer.state_dict().items()},
                             os.path.join(d, f"layer_{idx:02d}-model_{tp:02d}-model_states.pt"))
            _atomic_save({"module": None, **common}, os.path.join(d, f"mp_rank_{_mp_file_rank():02d}_model_states.pt"))
    elif writer:
        sd = {k: v.detach().cpu() for k, v in module.state_dict().items()}
        _atomic_save({"module": sd, **common}, os.path.join(d, f"mp_rank_{tp:02d}_model_states.pt"))
    if mpu.get_expert_parallel_world_size() > 1 and mpu.get_expert_data_parallel_rank() == 0:
        experts = _expert_params(module)
        if experts:
            _atomic_save({n: p.detach().cpu() for n, p in experts.items()}, _expert_file(d))
    if engine.optimizer is not None and not engine.neox_args.no_save_optim:
        if _per_rank_optimizer_state(engine) or writer:
            _atomic_save({"optimizer_state_dict": engine.optimizer.state_dict(),
                          "ds_config": engine.neox_args.deepspeed_config, "ds_version": "neox-b200"},
                         _optim_file(save_dir, tag, engine.neox_args.precision == "bfloat16"))
    _barrier()
    if _rank() == 0:
        # every rank has finished writing: mark the tag complete, then move ``latest`` (both atomically)
        with open(os.path.join(d, COMPLETE_MARKER), "w") as fh:
            fh.write("ok\n")
        tmp = os.path.join(save_dir, f"latest.tmp.{os.getpid()}")
        with open(tmp, "w") as fh:
            fh.write(tag)
        os.replace(tmp, os.path.join(save_dir, "latest"))
    _barrier()
    return True


def _load_module_sequential(module, sd, strict):
    missing, unexpected = module.load_state_dict(sd, strict=False)
    missing = [m for m in missing if "inv_freq" not in m]
    if strict and (missing or unexpected):
        raise RuntimeError(f"checkpoint mismatch; missing {missing[:5]}... unexpected {unexpected[:5]}...")


def engine_load_checkpoint(engine, load_dir, tag, load_optimizer_states, load_lr_scheduler_states, load_module_only,
                           load_module_strict):
    """Load ``tag`` (default: the tag named by ``latest``).  Without an explicit tag a damaged or missing newest
    checkpoint is not fatal: the newest tag whose save completed is used instead, with a message; if ``latest``
    itself is missing the newest completed tag is taken."""
    if tag is not None:
        return _load_tag(engine, load_dir, tag, load_optimizer_states, load_lr_scheduler_states, load_module_only,
                         load_module_strict)
    candidates = []
    latest = os.path.join(load_dir, "latest")
    if os.path.isfile(latest):
        with open(latest) as fh:
            candidates.append(fh.read().strip())
    else:
        found = complete_tags(load_dir)
        if found:
            print_rank_0(f" > {latest} is missing; newest completed checkpoint is {found[0]}")
    candidates += [t for t in complete_tags(load_dir) if t not in candidates]
    for i, cand in enumerate(candidates):
        err, got = None, (None, None)
        try:
            got = _load_tag(engine, load_dir, cand, load_optimizer_states, load_lr_scheduler_states, load_module_only,
                            load_module_strict)
        except (CheckpointDamaged, FileNotFoundError) as exc:
            err = exc
        # every rank reads its own files: all of them must agree before a tag is accepted
        if _all_ranks_ok(err is None):
            if got[0] is not None:
                return got
            continue
        nxt = candidates[i + 1] if i + 1 < len(candidates) else None
        why = err if err is not None else "another rank could not read its part"
        print(f" > [rank {_rank()}] checkpoint {cand} is unusable: {why}" +
              (f"\n > falling back to {nxt}" if nxt else "\n > no older completed checkpoint to fall back to"),
              flush=True)
        if nxt is None:
            raise err if err is not None else CheckpointDamaged(f"checkpoint {cand} is unreadable on another rank")
    return None, None


def _all_ranks_ok(ok: bool) -> bool:
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return ok
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    return bool(flag.item())


def _load_tag(engine, load_dir, tag, load_optimizer_states, load_lr_scheduler_states, load_module_only,
              load_module_strict):
    with _params_resident(engine):
        return _load_tag_impl(engine, load_dir, tag, load_optimizer_states, load_lr_scheduler_states,
                              load_module_only, load_module_strict)


def _load_tag_impl(engine, load_dir, tag, load_optimizer_states, load_lr_scheduler_states, load_module_only,
              load_module_strict):
    d = os.path.join(load_dir, tag)
    tp = mpu.get_model_parallel_rank()
    module = engine.module
    if _is_pipe_module(module):
        state_file = os.path.join(d, f"mp_rank_{_mp_file_rank():02d}_model_states.pt")
        if not os.path.isfile(state_file):
            state_file = os.path.join(d, f"mp_rank_{tp:02d}_model_states.pt")
        if not os.path.isfile(state_file):
            return None, None
        state = _read(state_file)
        for idx in module.local_layer_indices():
            layer = module.layer_module(idx)
            if layer is None or not any(True for _ in layer.state_dict()):
                continue
            f = os.path.join(d, f"layer_{idx:02d}-model_{tp:02d}-model_states.pt")
            if os.path.isfile(f):
                sd = _read(f)
            elif state.get("module") is not None:
                # a sequential-layout checkpoint read into a pipeline module: this layer's entries of the one state dict
                pre = f"sequential.{idx}."
                sd = {k[len(pre):]: v for k, v in state["module"].items() if k.startswith(pre)}
                if not sd and load_module_strict:
                    raise KeyError(f"{state_file} has no parameters of layer {idx}")
            elif load_module_strict:
                raise FileNotFoundError(f)
            else:
                continue
            _load_module_sequential(layer, sd, load_module_strict)
    else:
        state_file = os.path.join(d, f"mp_rank_{tp:02d}_model_states.pt")
        if not os.path.isfile(state_file):
            return None, None
        state = _read(state_file)
        if state.get("module") is not None:
            _load_module_sequential(module, state["module"], load_module_strict)
        else:
            # a pipeline-layout checkpoint read into a sequential model: one file per layer
            for idx, layer in enumerate(module.sequential):
                f = os.path.join(d, f"layer_{idx:02d}-model_{tp:02d}-model_states.pt")
                if os.path.isfile(f) and any(True for _ in layer.state_dict()):
                    _load_module_sequential(layer, _read(f),
                                            load_module_strict)
    if mpu.get_expert_parallel_world_size() > 1:
        experts = _expert_params(module)
        f = _expert_file(d)
        if experts and os.path.isfile(f):
            saved = _read(f)
            with torch.no_grad():
                for n, p in experts.items():
                    if n in saved:
                        p.copy_(saved[n].to(p.device))
                    elif load_module_strict:
                        raise KeyError(f"{f} has no entry for expert parameter {n}")
        elif experts and load_module_strict:
            raise FileNotFoundError(f"{f}: this run splits the experts over {mpu.get_expert_parallel_world_size()} "
                                    "ranks, but the checkpoint has no expert file for this rank")
    if engine.optimizer is not None and hasattr(engine.optimizer, "refresh_master_from_params"):
        engine.optimizer.refresh_master_from_params()
    if not load_module_only:
        engine.global_steps = state.get("global_steps", 0)
        engine.global_samples = state.get("global_samples", 0)
        engine.skipped_steps = state.get("skipped_steps", 0)
        if load_lr_scheduler_states and engine.lr_scheduler is not None and state.get("lr_scheduler") is not None:
            engine.lr_scheduler.load_state_dict(state["lr_scheduler"])
        if load_optimizer_states and engine.optimizer is not None:
            bf16 = engine.neox_args.precision == "bfloat16"
            # without ZeRO (and without experts of its own) every data-parallel rank holds the same optimizer
            # state and only rank 0 wrote it
            ranks = [None] if _per_rank_optimizer_state(engine) else [None, 0]
            cands = [_optim_file(load_dir, tag, b, r) for r in ranks for b in (bf16, not bf16)]
            f = next((c for c in cands if os.path.isfile(c)), cands[0])
            if os.path.isfile(f):
                osd = _read(f)
                engine.optimizer.load_state_dict(osd["optimizer_state_dict"])
            else:
                print_rank_0(f" > optimizer state file {f} not found; optimizer starts fresh")
    return d, state


# ------------------------------------------------------------------------------------ public API
def delete_old_checkpoints(save_dir, n_to_keep):
    if _rank() != 0:
        return
    pat = re.compile(r"global_step(\d+)$")
    found = [c for c in os.listdir(save_dir) if pat.match(c) and os.path.isdir(os.path.join(save_dir, c))]
    found = natural_sort(found)
    n_to_delete = len(found) - n_to_keep
    for c in found[:max(0, n_to_delete)]:
        try:
            shutil.rmtree(os.path.join(save_dir, c))
        except FileNotFoundError:
            pass


def save_ds_checkpoint(iteration, model, neox_args):
    sd = {"iteration": iteration, "args": {k: getattr(neox_args, k) for k in _CHECK_ARGS}}
    if not neox_args.no_save_rng:
        sd["random_rng_state"] = random.getstate()
        sd["np_rng_state"] = np.random.get_state()
        sd["torch_rng_state"] = torch.get_rng_state()
        sd["cuda_rng_state"] = torch.cuda.get_rng_state() if torch.cuda.is_available() else None
        sd["rng_tracker_states"] = get_cuda_rng_tracker().get_states()
    if neox_args.checkpoint_validation_with_forward_pass:
        sd["checkpoint_validation_logits"] = do_forward_pass(neox_args=neox_args, model=model)
    tag = get_checkpoint_tag(iteration)
    model.save_checkpoint(neox_args.save, tag=tag, client_state=sd)
    if _rank() == 0 and neox_args.config_files is not None:
        cdir = os.path.join(neox_args.save, tag, "configs")
        os.makedirs(cdir, exist_ok=True)
        for name, data in neox_args.config_files.items():
            with open(os.path.join(cdir, name), "w") as fh:
                fh.write(data) if isinstance(data, str) else json.dump(data, fh)


def upload_checkpoint(iteration, neox_args):
    """Mirror ``<save>/global_stepN`` to ``s3_path`` with multipart uploads (needs boto3)."""
    try:
        import boto3
        from boto3.s3.transfer import TransferConfig
    except ModuleNotFoundError:
        print("For s3 checkpointing, please install boto3 either using requirements/requirements-s3.txt or "
              "https://github.com/boto/boto3", file=sys.stderr)
        raise
    local = os.path.join(os.path.abspath(neox_args.save), get_checkpoint_tag(iteration))
    remote = os.path.join(neox_args.s3_path, os.path.basename(neox_args.save), get_checkpoint_tag(iteration))
    m = re.match(r"s3://([^/]+)/?(.*)", remote)
    bucket, prefix = m.group(1), m.group(2)
    cfg = TransferConfig(multipart_threshold=neox_args.s3_chunk_size, multipart_chunksize=neox_args.s3_chunk_size,
                         max_concurrency=8, use_threads=True)
    s3 = boto3.client("s3")
    for root, _, files in os.walk(local):
        for name in files:
            path = os.path.join(root, name)
            key = os.path.join(prefix, os.path.relpath(path, local))
            s3.upload_file(path, bucket, key, Config=cfg)
    print_rank_0(f"[RANK 0] uploaded checkpoint `{local}` to `{remote}`")


def save_checkpoint(neox_args, iteration, model, optimizer, lr_scheduler):
    if neox_args.deepspeed:
        save_ds_checkpoint(iteration, model, neox_args)
    else:
        raise ValueError("Must be using deepspeed to use neox")
    _barrier()
    if neox_args.s3_path is not None and _rank() == 0:
        upload_checkpoint(iteration, neox_args)
    _barrier()
    if neox_args.keep_last_n_checkpoints is not None:
        delete_old_checkpoints(neox_args.save, neox_args.keep_last_n_checkpoints)
    _barrier()


def load_checkpoint(neox_args, model, optimizer, lr_scheduler, inference=False, iteration=None):
    """Load a checkpoint; returns the iteration to resume from (0 when nothing was found or
    ``finetune`` is set)."""
    if not neox_args.deepspeed:
        raise ValueError("Must be using deepspeed to use neox")
    load_optim_and_scheduler = not neox_args.no_load_optim
    tag = get_checkpoint_tag(iteration) if iteration is not None else None
    path, state = model.load_checkpoint(neox_args.load, load_optimizer_states=load_optim_and_scheduler,
                                        load_lr_scheduler_states=load_optim_and_scheduler,
                                        load_module_only=not load_optim_and_scheduler, tag=tag,
                                        load_module_strict=neox_args.train_impl != "rm")
    if path is None:
        if iteration is not None:
            available = sorted(int(i.name.replace("global_step", "")) for i in os.scandir(neox_args.load)
                               if i.is_dir() and i.name.startswith("global_step")) if os.path.isdir(neox_args.load) else []
            raise ValueError(f"Unable to load checkpoint for iteration {iteration}. \nAvailable iterations: {available}")
        if mpu.get_data_parallel_rank() == 0:
            print("Unable to load checkpoint.")
        return 0
    if neox_args.finetune:
        iteration = 0
    else:
        iteration = state.get("iteration", state.get("total_iters", 0))
    if "args" in state:
        check_checkpoint_args(neox_args=neox_args, checkpoint_args=state["args"])
    else:
        print_rank_0(" > could not find arguments in the checkpoint for validation...")
    if neox_args.checkpoint_validation_with_forward_pass and "checkpoint_validation_logits" in state:
        check_forward_pass(neox_args=neox_args, model=model,
                           checkpoint_logits=state["checkpoint_validation_logits"], inference=inference)
    if not neox_args.finetune and not neox_args.no_load_rng:
        try:
            random.setstate(state["random_rng_state"])
            np.random.set_state(state["np_rng_state"])
            torch.set_rng_state(state["torch_rng_state"])
            if torch.cuda.is_available() and state.get("cuda_rng_state") is not None:
                torch.cuda.set_rng_state(state["cuda_rng_state"])
            get_cuda_rng_tracker().set_states(state["rng_tracker_states"])
        except KeyError:
            print_rank_0(f"Unable to load rngs from checkpoint {path}, exiting. Specify --no-load-rng or --finetune "
                         "to prevent attempting to load the random state.")
            sys.exit()
    _barrier()
    if mpu.get_data_parallel_rank() == 0:
        print(f"  successfully loaded {path}")
    return iteration
