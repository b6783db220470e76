"""General helpers (role of ``megatron/utils.py`` in the reference): rank-aware printing, mask and
position-id construction, loss reduction, timers, overflow monitor, parameter counting and the
inference/eval bootstrap."""
from __future__ import annotations

import os
import re
import sys
import time
from typing import Dict, List

import torch
import torch.distributed as dist

from ..parallel import mpu


def _dist_on():
    return dist.is_available() and dist.is_initialized()


def is_rank_0():
    return not _dist_on() or dist.get_rank() == 0


def is_local_main():
    return local_rank() == 0


def is_mp_rank_0():
    return mpu.get_model_parallel_rank() == 0


def print_rank_0(*message):
    if is_rank_0():
        print(*message, flush=True)


def local_rank():
    v = os.environ.get("LOCAL_RANK", os.environ.get("SLURM_LOCALID"))
    return int(v) if v is not None else 0


def natural_sort(items):
    conv = lambda t: int(t) if t.isdigit() else t.lower()
    return sorted(items, key=lambda k: [conv(c) for c in re.split("([0-9]+)", k)])


def ddb(rank=0):
    """Drop into pdb on one rank, everybody else waits at a barrier."""
    if not _dist_on() or dist.get_rank() == rank:
        from pdb import Pdb
        Pdb(skip=["torch.distributed.*"]).set_trace(sys._getframe().f_back)
    if _dist_on():
        dist.barrier()


def get_attn_mask(seq_length, device, sliding_window_width=None):
    """Boolean ``[1, 1, s, s]`` mask, True where attention is NOT allowed."""
    i = torch.arange(seq_length, device=device)
    mask = i[None, :] > i[:, None]
    if sliding_window_width is not None:
        mask = mask | (i[None, :] < i[:, None] - sliding_window_width)
    return mask.view(1, 1, seq_length, seq_length)


def get_ltor_masks_and_position_ids(data, eod_token, eod_mask_loss=False, sliding_window_width=None,
                                    build_attention_mask=False):
    """Loss mask, position ids and (only when asked: the kernels generate causal / sliding-window masks
    themselves) the dense attention mask for a left-to-right model."""
    batch_size, seq_length = data.size()
    attention_mask = get_attn_mask(seq_length, data.device, sliding_window_width) if build_attention_mask else None
    loss_mask = torch.ones(data.size(), dtype=torch.float, device=data.device)
    if eod_mask_loss:
        loss_mask[data == eod_token] = 0.0
    position_ids = torch.arange(seq_length, dtype=torch.long, device=data.device).unsqueeze(0).expand_as(data)
    return attention_mask, loss_mask, position_ids


def reduce_losses(losses):
    """Average a list of scalar losses over all ranks."""
    red = torch.cat([l.clone().detach().view(1).float() for l in losses])
    if _dist_on():
        dist.all_reduce(red)
        red = red / dist.get_world_size()
    return red


def report_memory(name):
    if not torch.cuda.is_available():
        return
    mb = 1024.0 * 1024.0
    print_rank_0(f"{name} memory (MB) | allocated: {torch.cuda.memory_allocated() / mb} | max allocated: "
                 f"{torch.cuda.max_memory_allocated() / mb} | reserved: {torch.cuda.memory_reserved() / mb} | "
                 f"max reserved: {torch.cuda.max_memory_reserved() / mb}")


def get_total_params(model):
    """Parameter count over the whole model-parallel grid (counted on data-parallel rank 0)."""
    if mpu.get_data_parallel_rank() == 0:
        n = sum(p.nelement() for p in model.parameters())
    else:
        n = 0
    dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    t = torch.tensor([n], dtype=torch.int64, device=dev)
    if _dist_on():
        dist.all_reduce(t)
    return int(t.item())


class Timer:
    """Accumulating timer.  On CUDA it records events on the current stream and resolves the elapsed
    time lazily, so ``start``/``stop`` do not synchronise the device (the reference's timers call
    ``torch.cuda.synchronize()`` twice per region, ``megatron/utils.py:239-251``)."""

    def __init__(self, name):
        self.name_ = name
        self.elapsed_ = 0.0
        self.started_ = False
        self._pairs = []
        self._t0 = None
        self._cuda = torch.cuda.is_available()

    def start(self):
        assert not self.started_, "timer has already been started"
        if self._cuda:
            self._t0 = torch.cuda.Event(enable_timing=True)
            self._t0.record()
        else:
            self._t0 = time.time()
        self.started_ = True

    def stop(self):
        assert self.started_, "timer is not started"
        if self._cuda:
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            self._pairs.append((self._t0, e))
        else:
            self.elapsed_ += time.time() - self._t0
        self.started_ = False

    def reset(self):
        self.elapsed_, self.started_, self._pairs = 0.0, False, []

    def elapsed(self, reset=True):
        was = self.started_
        if was:
            self.stop()
        if self._pairs:
            self._pairs[-1][1].synchronize()
            self.elapsed_ += sum(a.elapsed_time(b) for a, b in self._pairs) / 1000.0
            self._pairs = []
        out = self.elapsed_
        if reset:
            self.reset()
        if was:
            self.start()
        return out


class Timers:
    def __init__(self, use_wandb=False, tensorboard_writer=None, comet_experiment=None):
        self.timers = {}
        self.use_wandb, self.tensorboard_writer, self.comet_experiment = use_wandb, tensorboard_writer, comet_experiment

    def __call__(self, name):
        if name not in self.timers:
            self.timers[name] = Timer(name)
        return self.timers[name]

    def write(self, names, iteration, normalizer=1.0, reset=False):
        assert normalizer > 0.0
        for name in names:
            value = self.timers[name].elapsed(reset=reset) / normalizer
            if self.tensorboard_writer:
                self.tensorboard_writer.add_scalar(f"timers/{name}", value, iteration)
            if self.use_wandb:
                import wandb
                wandb.log({f"timers/{name}": value}, step=iteration)
            if self.comet_experiment:
                self.comet_experiment.__internal_api__log_metric__(f"timers/{name}", value, framework="neox-b200",
                                                                   step=iteration)

    def log(self, names, normalizer=1.0, reset=True):
        assert normalizer > 0.0
        string = "time (ms)"
        for name in names:
            string += " | {}: {:.2f}".format(name, self.timers[name].elapsed(reset=reset) * 1000.0 / normalizer)
        print_rank_0(string)


class OverflowMonitor:
    """Abort when fp16 overflow skipped ``n`` optimizer steps in a row (``megatron/utils.py:356-380``)."""

    def __init__(self, optimizer, n=50):
        self.optimizer, self.n = optimizer, n
        self.history = []

    def check(self, skipped):
        self.history.append(bool(skipped))
        self.history = self.history[-self.n:]
        scale = getattr(self.optimizer, "cur_scale", None)
        dynamic = getattr(getattr(self.optimizer, "loss_scaler", None), "dynamic", False)
        if dynamic and len(self.history) == self.n and all(self.history) and scale is not None and scale <= \
                getattr(self.optimizer.loss_scaler, "min_scale", 1.0):
            raise Exception(f"Skipped {self.n} iterations in a row due to Overflow - Exiting training.")


def get_noise_scale_logger(neox_args):
    if neox_args.log_gradient_noise_scale:
        if neox_args.zero_stage >= 1:
            raise NotImplementedError("Gradient Noise Scale logging does not work with zero stage 2+, as the "
                                      "gradients are distributed across ranks.")
        from ..gradient_noise_scale import GradientNoiseScale
        return lambda model: GradientNoiseScale(model=model, batch_size_small=neox_args.train_batch_size,
                                                n_batches=neox_args.gradient_noise_scale_n_batches,
                                                cpu_offload=neox_args.gradient_noise_scale_cpu_offload,
                                                neox_args=neox_args, mpu=mpu)
    return None


class CharCounter:
    """Wraps a data iterator and counts characters of the decoded batches (char-level perplexity)."""

    def __init__(self, data_iterator, tokenizer):
        self.tokenizer, self.data_iterator = tokenizer, data_iterator
        self.char_count, self.batch_count, self.token_count, self.total_time = 0, 0, 0, 0.0

    def tokens_per_char(self):
        return self.token_count / max(self.char_count, 1)

    def __iter__(self):
        return self

    def __next__(self):
        t0 = time.time()
        batch = next(self.data_iterator)
        for b in batch["text"]:
            self.token_count += len(b)
            self.char_count += len(self.tokenizer.detokenize(b.tolist()))
        self.batch_count += 1
        self.total_time += time.time() - t0
        return batch


def get_deepspeed_config(neox_args):
    return neox_args.deepspeed_config


def setup_for_inference_or_eval(use_cache=True, overwrite_values=None, input_args=None):
    """Build args, model and load the checkpoint for generation / evaluation
    (``megatron/utils.py:422-469``): no activation checkpointing, no optimizer, no ZeRO."""
    from ..config import NeoXArgs
    from ..initialize import initialize_megatron
    from ..training import setup_model_and_optimizer

    overwrite = {"checkpoint_activations": False, "partition_activations": False, "no_load_optim": True,
                 "optimizer": None, "zero_optimization": None}
    if overwrite_values:
        overwrite.update(overwrite_values)
    neox_args = NeoXArgs.consume_neox_args(overwrite_values=overwrite, input_args=input_args)
    neox_args.configure_distributed_args()
    neox_args.build_tokenizer()
    if neox_args.load is None:
        raise ValueError("`load` parameter must be supplied to load a model`")
    initialize_megatron(neox_args)
    model, _, _, _ = setup_model_and_optimizer(neox_args=neox_args, use_cache=use_cache, iteration=neox_args.iteration)
    print_rank_0("Finished loading model")
    model.module.inference_mode(use_cache=use_cache)
    return model, neox_args
