"""Autotuner: short trial runs over micro-batch size and ZeRO stage, pick the fastest configuration.

``deepy.py train.py cfg.yml --autotuning tune`` runs the trials and writes their results; ``--autotuning run`` then
also starts the real job with the winning values.  The reference hands this job to DeepSpeed's autotuner through the
same flag and the ``autotuning`` block (``megatron/neox_arguments/arguments.py:495-503``; block keys as in
``configs/autotuning_configs/*.json``: ``enabled, start_profile_step, end_profile_step, metric, fast,
max_train_batch_size, min/max_train_micro_batch_size_per_gpu, num_tuning_micro_batch_sizes, tuner_type,
tuner_early_stopping, tuner_num_trials, results_dir, exps_dir, overwrite``).

A trial is the ordinary training job, launched by the ordinary launcher, with ``train_iters`` cut to
``end_profile_step + 1``, checkpointing and evaluation off, and ``autotuning_metric_path`` pointing at a file into
which the training loop writes the throughput it measured between the two profile steps.  A trial that dies (out of
memory, usually) has no metric file: larger micro-batches of the same ZeRO stage are then skipped.
"""
from __future__ import annotations

import copy
import json
import os
import random

METRICS = {"throughput": ("throughput", True), "latency": ("latency", False), "flops": ("tokens_per_sec", True)}


class Autotuner:
    def __init__(self, neox_args, runner=None):
        """``runner(trial_args) -> exit code`` launches one trial (default: ``launcher.launch``)."""
        self.args = neox_args
        self.block = dict(neox_args.autotuning or {})
        self.runner = runner
        self.results_dir = self.block.get("results_dir") or "autotuning_results"
        self.exps_dir = self.block.get("exps_dir") or "autotuning_exps"
        metric = str(self.block.get("metric", "throughput")).lower()
        self.metric_key, self.higher_is_better = METRICS.get(metric, METRICS["throughput"])
        self.records = []

    # ------------------------------------------------------------------ search space
    def micro_batch_sizes(self):
        lo = int(self.block.get("min_train_micro_batch_size_per_gpu", 1))
        hi = int(self.block.get("max_train_micro_batch_size_per_gpu", 1024))
        n = int(self.block.get("num_tuning_micro_batch_sizes", 3))
        cap = self.block.get("max_train_batch_size")
        dp = max(int(self.args.dp_world_size or 1), 1)
        out, mb = [], max(lo, 1)
        while mb <= hi and len(out) < n:
            if cap is not None and mb * dp > int(cap):
                break
            out.append(mb)
            mb *= 2
        return out or [max(lo, 1)]

    def zero_stages(self):
        zero = self.args.zero_optimization or {}
        stage = zero.get("stage", 0)
        if stage == "auto" or self.block.get("tune_zero_stage", False):
            # gradient / parameter partitioning (2, 3) is not available under pipeline parallelism
            return [0, 1] if (self.args.pipe_parallel_size or 0) >= 1 else [0, 1, 2, 3]
        return [int(stage)]

    def experiments(self):
        exps = [{"zero_stage": z, "micro_batch": mb} for z in self.zero_stages() for mb in self.micro_batch_sizes()]
        if str(self.block.get("tuner_type", "gridsearch")).lower() == "random":
            random.Random(int(self.block.get("seed", 0))).shuffle(exps)
        limit = int(self.block.get("tuner_num_trials", len(exps)))
        return exps[:limit]

    # ------------------------------------------------------------------ one trial
    def trial_args(self, exp, metric_path):
        from .config import NeoXArgs
        cfg = copy.deepcopy(self.args.all_config)
        dp = max(int(self.args.dp_world_size or 1), 1)
        gas = int(self.block.get("gradient_accumulation_steps", 1))
        zero = dict(cfg.get("zero_optimization") or {})
        zero["stage"] = exp["zero_stage"]
        block = dict(self.block, enabled=False)
        cfg.update({
            "train_micro_batch_size_per_gpu": exp["micro_batch"], "gradient_accumulation_steps": gas,
            "train_batch_size": exp["micro_batch"] * gas * dp, "zero_optimization": zero,
            "train_iters": int(self.block.get("end_profile_step", 5)) + 1, "lr_decay_iters": None,
            "save": None, "load": None, "eval_interval": 10 ** 9, "do_valid": False, "do_test": False,
            "checkpoint_factor": 10 ** 9, "autotuning_run": None, "autotuning": block,
            "autotuning_metric_path": metric_path, "use_wandb": False, "tensorboard_dir": None,
        })
        cfg = {k: v for k, v in cfg.items() if v is not None}
        return NeoXArgs.from_dict(cfg)

    def run_trial(self, exp):
        name = f"z{exp['zero_stage']}_mbs{exp['micro_batch']}"
        exp_dir = os.path.join(self.exps_dir, name)
        os.makedirs(exp_dir, exist_ok=True)
        metric_path = os.path.join(exp_dir, "metric.json")
        if os.path.exists(metric_path):
            if self.block.get("overwrite", True):
                os.remove(metric_path)
            else:
                with open(metric_path) as fh:
                    return {"name": name, **exp, "exit_code": 0, **json.load(fh), "reused": True}
        args = self.trial_args(exp, metric_path)
        runner = self.runner
        if runner is None:
            from .launcher import launch
            runner = launch
        code = runner(args)
        rec = {"name": name, **exp, "exit_code": int(code or 0)}
        if os.path.exists(metric_path):
            with open(metric_path) as fh:
                rec.update(json.load(fh))
        return rec

    # ------------------------------------------------------------------ the search
    def better(self, a, b):
        if b is None:
            return True
        return a > b if self.higher_is_better else a < b

    def tune(self):
        """Run the trials; returns the best record (``None`` when every trial failed) and writes
        ``<results_dir>/summary.json`` and ``summary.txt``."""
        os.makedirs(self.results_dir, exist_ok=True)
        patience = int(self.block.get("tuner_early_stopping", 5))
        best, since_best, failed_stage = None, 0, {}
        for exp in self.experiments():
            # a stage that already ran out of memory will not fit a larger micro-batch either
            if failed_stage.get(exp["zero_stage"], 10 ** 9) <= exp["micro_batch"]:
                self.records.append({"name": f"z{exp['zero_stage']}_mbs{exp['micro_batch']}", **exp, "skipped": True})
                continue
            rec = self.run_trial(exp)
            self.records.append(rec)
            value = rec.get(self.metric_key)
            if value is None:
                failed_stage[exp["zero_stage"]] = min(failed_stage.get(exp["zero_stage"], 10 ** 9), exp["micro_batch"])
                continue
            if self.better(value, best.get(self.metric_key) if best else None):
                best, since_best = rec, 0
            else:
                since_best += 1
                if since_best >= patience:
                    break
        with open(os.path.join(self.results_dir, "summary.json"), "w") as fh:
            json.dump({"metric": self.metric_key, "best": best, "experiments": self.records}, fh, indent=1)
        with open(os.path.join(self.results_dir, "summary.txt"), "w") as fh:
            fh.write(self.summary(best))
        print(self.summary(best), flush=True)
        return best

    def summary(self, best):
        lines = [f"autotuning: {len(self.records)} experiment(s), metric {self.metric_key}",
                 f"{'experiment':<18}{'zero':<6}{'micro-batch':<13}{self.metric_key:<16}status"]
        for r in self.records:
            value = r.get(self.metric_key)
            status = "skipped" if r.get("skipped") else ("ok" if value is not None else f"failed ({r.get('exit_code')})")
            lines.append(f"{r['name']:<18}{r['zero_stage']:<6}{r['micro_batch']:<13}"
                         f"{(f'{value:.3f}' if value is not None else '-'):<16}{status}")
        lines.append(f"best: {best['name']}" if best else "best: none (every trial failed)")
        return "\n".join(lines) + "\n"

    def apply_best(self, best):
        """The job's own arguments with the winning micro-batch and ZeRO stage (global batch kept when it divides)."""
        from .config import NeoXArgs
        cfg = copy.deepcopy(self.args.all_config)
        dp = max(int(self.args.dp_world_size or 1), 1)
        zero = dict(cfg.get("zero_optimization") or {})
        zero["stage"] = best["zero_stage"]
        mb = best["micro_batch"]
        tb = cfg.get("train_batch_size") or mb * dp
        gas = max(tb // (mb * dp), 1)
        cfg.update({"train_micro_batch_size_per_gpu": mb, "gradient_accumulation_steps": gas,
                    "train_batch_size": mb * gas * dp, "zero_optimization": zero, "autotuning_run": None})
        return NeoXArgs.from_dict({k: v for k, v in cfg.items() if v is not None})
