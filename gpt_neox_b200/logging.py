"""Metrics and console/TensorBoard/W&B/Comet logging (role of ``megatron/logging.py``).

The FLOPs model is the reference's *definition* of the headline metrics, so it is reproduced as a
formula (``megatron/logging.py:83-237``):

    transformer:  24 * c * B * s * L * h^2 * (1 + s/(6h) + V/(16 L h))
    rwkv:         B * s * (78 h^2 L + 84 h L + 16 h + 12 h V + 18 h^2 L / heads)
    mamba:        L * c * B * s * d_in * (11 d_state + 4 dt_rank + 1 + 6 h + 2 d_conv) + 6 B s h V

``c`` = 3 for model FLOPs (MFU) and 4 for hardware FLOPs when activation checkpointing is on (HFU).
``tokens_per_sec = train_batch_size * seq_length / iteration_time``.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist

from .utils import print_rank_0, report_memory


def flops_per_iteration(neox_args, factor) -> float:
    V, B, s, h, L = (neox_args.padded_vocab_size, neox_args.train_batch_size, neox_args.seq_length,
                     neox_args.hidden_size, neox_args.num_layers)
    kinds = neox_args.attention_config or []
    if "rwkv" in kinds:
        nh = neox_args.num_attention_heads
        return B * s * (78 * h * h * L + 84 * h * L + 16 * h + 12 * h * V + 18 * h * h * L / nh)
    if "mamba" in kinds:
        if neox_args.expansion_factor:
            d_in = h * neox_args.expansion_factor
        elif neox_args.intermediate_size:
            d_in = neox_args.intermediate_size
        else:
            d_in = 2 * h
        d_state, d_conv, dt_rank = 16, 4, math.ceil(h / 16)
        per_layer = factor * s * B * d_in * ((11 * d_state + 4 * dt_rank + 1) + 6 * h + 2 * d_conv)
        return per_layer * L + 6 * s * B * h * V
    return 24 * factor * B * s * L * h * h * (1.0 + s / (6.0 * h) + V / (16.0 * L * h))


def _world():
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def get_actual_flops(neox_args, iter_time_s) -> float:
    """Hardware FLOP/s per GPU (recompute counted when activation checkpointing is on)."""
    return flops_per_iteration(neox_args, 4 if neox_args.checkpoint_activations else 3) / (iter_time_s * _world())


def get_forward_backward_flops(neox_args, iter_time_s) -> float:
    """Model FLOP/s per GPU (forward + backward only)."""
    return flops_per_iteration(neox_args, 3) / (iter_time_s * _world())


def human_readable_flops(num) -> str:
    for unit in ["", "KFLOPS", "MFLOPS", "GFLOPS", "TFLOPS", "PFLOPS", "EFLOPS", "ZFLOPS"]:
        if abs(num) < 1000.0:
            return "%3.1f%s" % (num, unit)
        num /= 1000.0
    return "%.1f%s" % (num, "Yi")


class CsvMonitor:
    """The ``csv_monitor`` block of the DeepSpeed configuration (``{"enabled": true, "output_path": ..., "job_name":
    ...}``): every scalar goes to ``<output_path>/<job_name>/<key with / as _>.csv`` as ``step,value`` lines."""

    def __init__(self, cfg):
        cfg = cfg or {}
        self.enabled = bool(cfg.get("enabled", False))
        self.dir = os.path.join(cfg.get("output_path") or "csv_monitor", cfg.get("job_name") or "DeepSpeedJobName")
        self._files = {}

    def log(self, key, value, step):
        if not self.enabled:
            return
        fh = self._files.get(key)
        if fh is None:
            os.makedirs(self.dir, exist_ok=True)
            path = os.path.join(self.dir, key.replace("/", "_").replace(" ", "_") + ".csv")
            new = not os.path.exists(path)
            fh = self._files[key] = open(path, "a", buffering=1)
            if new:
                fh.write(f"step,{key}\n")
        fh.write(f"{int(step)},{float(value)}\n")

    def close(self):
        for fh in self._files.values():
            fh.close()
        self._files = {}


_csv_monitor = CsvMonitor(None)


def configure_csv_monitor(cfg):
    """Install the CSV sink that ``tb_wandb_log`` also writes to (rank 0); returns it."""
    global _csv_monitor
    _csv_monitor.close()
    _csv_monitor = CsvMonitor(cfg)
    return _csv_monitor


def tb_wandb_log(key, value, iteration_no, use_wandb, tensorboard_writer=None, comet_experiment=None,
                 all_ranks=False):
    """Send one scalar to every enabled sink (rank 0 only unless ``all_ranks``)."""
    do_log = (dist.get_rank() == 0 if dist.is_available() and dist.is_initialized() else True) or all_ranks
    if not do_log or value is None:
        return
    _csv_monitor.log(key, value, iteration_no)
    if tensorboard_writer:
        tensorboard_writer.add_scalar(key, value, iteration_no)
    if use_wandb:
        import wandb
        wandb.log({key: value}, step=iteration_no)
    if comet_experiment:
        comet_experiment.__internal_api__log_metric__(key, value, framework="neox-b200", step=iteration_no)


def _norm_logs(model, neox_args):
    out = {}
    if not (neox_args.log_grad_norm or neox_args.log_param_norm or neox_args.log_grad_pct_zeros):
        return out
    for name, p in model.module.named_parameters():
        g = getattr(p, "main_grad", None)
        if neox_args.log_grad_norm and g is not None:
            out[f"gradient_norms/{name}"] = g.float().norm().item()
        if neox_args.log_grad_pct_zeros and g is not None:
            out[f"pct_grad_zeros/{name}"] = (g == 0).float().mean().item() * 100
        if neox_args.log_param_norm:
            out[f"parameter_norms/{name}"] = p.detach().float().norm().item()
    return out


def training_log(neox_args, timers, loss_dict, total_loss_dict, learning_rate, iteration, loss_scale,
                 report_memory_flag, skipped_iter, model, optimizer, noise_scale_logger):
    """Accumulate losses, write scalars, and every ``log_interval`` iterations print the console line
    with throughput, FLOPs and utilisation."""
    skipped_key, nan_key = "skipped iterations", "got nan"
    total_loss_dict[skipped_key] = total_loss_dict.get(skipped_key, 0) + skipped_iter
    got_nan = False
    for key, val in loss_dict.items():
        v = float(val)
        is_bad = math.isinf(v) or math.isnan(v)
        got_nan = got_nan or is_bad
        if not skipped_iter and not is_bad:
            total_loss_dict[key] = total_loss_dict.get(key, 0.0) + v
    total_loss_dict[nan_key] = total_loss_dict.get(nan_key, 0) + int(got_nan)

    log = lambda k, v: tb_wandb_log(k, v, iteration, neox_args.use_wandb, neox_args.tensorboard_writer,
                                    neox_args.comet_experiment)
    # per-phase engine times (``wall_clock_breakdown``): fresh every ``steps_per_print`` optimizer steps
    if getattr(model, "timer_values", None) and model.wall_clock_breakdown() and \
            model.global_steps % model.steps_per_print() == 0:
        for key, val in model.timer_values.items():
            log(f"timers/{key}", val)
    log("train/learning_rate", learning_rate)
    for key, val in loss_dict.items():
        log(f"train/{key.replace(' ', '_')}", float(val))
    if neox_args.precision == "fp16":
        log("train/loss_scale", loss_scale)
    if noise_scale_logger is not None and getattr(noise_scale_logger, "noise_scale", None) is not None:
        log("train/noise_scale", noise_scale_logger.noise_scale)
    for k, v in _norm_logs(model, neox_args).items():
        log(k, v)
    if neox_args.log_optimizer_states and optimizer is not None:
        inner = getattr(optimizer, "optimizer", optimizer)
        for gi, state in enumerate(inner.state.values()):
            for sk, sv in state.items():
                if torch.is_tensor(sv) and sv.is_floating_point():
                    log(f"optimizer_state_norms/group{gi}_{sk}", sv.float().norm().item())

    if iteration % neox_args.log_interval == 0:
        elapsed = timers("interval time").elapsed()
        iter_time = elapsed / neox_args.log_interval
        samples_per_sec = neox_args.train_batch_size / iter_time
        steps_per_sec = 1.0 / iter_time
        tokens_per_sec = samples_per_sec * neox_args.seq_length
        log_string = " samples/sec: {:.3f} |".format(samples_per_sec)
        log("runtime/samples_per_sec", samples_per_sec)
        log("runtime/iteration_time", iter_time)
        log("runtime/steps_per_sec", steps_per_sec)
        log("runtime/tokens_per_sec", tokens_per_sec)
        log_string += " iteration {:8d}/{:8d} |".format(iteration, neox_args.train_iters)
        log_string += " elapsed time per iteration (ms): {:.1f} |".format(iter_time * 1000.0)
        log_string += " learning rate: {:.3E} |".format(learning_rate)
        num_iterations = max(1, neox_args.log_interval - total_loss_dict[skipped_key])
        avg_time = iter_time
        for key in list(total_loss_dict.keys()):
            if key in (skipped_key, nan_key):
                continue
            v = total_loss_dict[key]
            avg = float(v) / num_iterations
            log_string += " {}: {:.6E} |".format(key, avg)
            total_loss_dict[key] = 0.0
        if neox_args.precision == "fp16":
            log_string += " loss scale: {:.1f} |".format(loss_scale)
        log_string += " number of skipped iterations: {:3d} |".format(total_loss_dict[skipped_key])
        log_string += " number of nan iterations: {:3d} |".format(total_loss_dict[nan_key])
        total_loss_dict[skipped_key] = 0
        total_loss_dict[nan_key] = 0
        flops_per_s_per_gpu = get_actual_flops(neox_args, iter_time)
        fb_flops = get_forward_backward_flops(neox_args, iter_time)
        log_string += " approx flops per GPU: {} |".format(human_readable_flops(flops_per_s_per_gpu))
        log_string += " tokens/sec: {:.1f} |".format(tokens_per_sec)
        log("runtime/flops_per_sec_per_gpu", flops_per_s_per_gpu)
        if neox_args.peak_theoretical_tflops:
            peak = neox_args.peak_theoretical_tflops * 1e12
            mfu, hfu = fb_flops / peak * 100, flops_per_s_per_gpu / peak * 100
            log("runtime/model_flops_utilization", mfu)
            log("runtime/hardware_flops_utilization", hfu)
            log_string += " MFU: {:.2f}% approx flops per GPU: {} |".format(mfu, human_readable_flops(fb_flops))
            log_string += " HFU: {:.2f}% |".format(hfu)
        print_rank_0(log_string)
        if report_memory_flag:
            report_memory("after {} iterations".format(iteration))
            report_memory_flag = False
        if timers is not None:
            names = [n for n in ("forward", "backward", "backward-backward", "backward-allreduce",
                                 "backward-master-grad", "backward-clip-grad", "optimizer", "batch generator",
                                 "data loader") if n in timers.timers]
            if names:
                # the timers hold CUDA events that are resolved here, once per interval, not at every step
                if not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0:
                    timers.write(names, iteration, normalizer=neox_args.log_interval)
                timers.log(names, normalizer=neox_args.log_interval)
    return report_memory_flag
