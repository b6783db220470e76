"""``NeoXArgs``: one object holding every configuration value of a run.

Behavioural contract (reference: ``megatron/neox_arguments/arguments.py``):

* built from one or more YAML files that are merged (``from_ymls``; a key present in two files is an
  error; ``-`` and ``_`` are interchangeable in key names; unknown keys are rejected),
  from a dict (``from_dict``), from the launcher command line (``consume_deepy_args``) or from the
  base64-JSON blob the launcher hands every worker (``consume_neox_args``);
* ``calculate_derived`` solves the batch triple ``train_batch = micro * grad_acc * dp_world``, derives
  precision from the ``fp16`` / ``bf16`` blocks, fills ZeRO and optimizer defaults, expands
  ``attention_config`` to one entry per layer and applies the MoE / GQA / RWKV / Mamba exclusions;
* ``validate_types`` / ``validate_values`` reject ill-typed or inconsistent configurations;
* ``deepspeed_config`` is the engine-level sub-dict (non-default values only) and
  ``get_deepspeed_main_args`` is the worker argv.

The class is generated from the table in ``schema.py`` instead of being written as dataclasses.
"""
from __future__ import annotations

import argparse
import base64
import copy
import json
import logging
import os
import subprocess
import sys
from pathlib import Path
from socket import gethostname

import torch
import yaml

from .schema import (ATTENTION_TYPE_CHOICES, ENGINE_KEYS, FIELDS, OPT_DEFAULT, OPT_PARAMS_DEFAULTS,
                     RUNNER_KEYS, ZERO_DEFAULTS)

DLTS_HOSTFILE = "/job/hostfile"
AUTOTUNING_ARGS = ("train_batch_size", "train_micro_batch_size_per_gpu", "gradient_accumulation_steps",
                   "zero_optimization", "autotuning")
_TRANSIENT = ("tokenizer", "tensorboard_writer", "adlr_autoresume_object")


def git_commit_hash() -> str | None:
    try:
        out = subprocess.run(["git", "describe", "--always"], capture_output=True, text=True,
                             cwd=Path(__file__).resolve().parent, timeout=5)
        return out.stdout.strip() or None
    except Exception:
        return None


def expand_attention_types(attention_config, num_layers):
    """``[[["global","local"], 2], [["flash"], "all"]]`` -> flat list with one kind per layer."""
    if all(isinstance(i, str) for i in attention_config):
        return list(attention_config)
    out = []
    for kinds, repeat in attention_config:
        if repeat == "all":
            assert num_layers % len(kinds) == 0, \
                f"num_layers ({num_layers}) is not divisible by the length of the attention pattern {kinds}"
            return [kinds[i % len(kinds)] for i in range(num_layers)]
        for _ in range(int(repeat)):
            out.extend(kinds)
    return out


def read_hostfile(path):
    """``host slots=N`` lines -> ordered ``{host: N}`` (MPI-style hostfile)."""
    pool = {}
    with open(path) as fh:
        for line in fh:
            line = line.split("#", 1)[0].strip()
            if not line:
                continue
            try:
                host, slots = line.split()
                key, count = slots.split("=")
                assert key == "slots"
                pool[host] = int(count)
            except Exception as exc:
                raise ValueError(f"hostfile line not of the form 'host slots=N': {line!r}") from exc
    return pool


def _parse_filter(spec):
    """``'hostA:0,1@hostB'`` -> ``{'hostA': [0, 1], 'hostB': None}``."""
    out = {}
    for part in filter(None, spec.split("@")):
        if ":" in part:
            host, ids = part.split(":")
            out[host] = [int(i) for i in ids.split(",")]
        else:
            out[part] = None
    return out


def resource_pool(hostfile, include="", exclude=""):
    """Apply ``--include`` / ``--exclude`` filters to a hostfile; returns ``{host: [device ids]}``."""
    pool = {h: list(range(n)) for h, n in read_hostfile(hostfile).items()}
    if include and exclude:
        raise ValueError("include and exclude are mutually exclusive")
    if include:
        inc = _parse_filter(include)
        pool = {h: (ids if inc[h] is None else [i for i in ids if i in inc[h]]) for h, ids in pool.items() if h in inc}
    elif exclude:
        exc = _parse_filter(exclude)
        kept = {}
        for h, ids in pool.items():
            if h in exc:
                if exc[h] is None:
                    continue
                ids = [i for i in ids if i not in exc[h]]
            if ids:
                kept[h] = ids
        pool = kept
    return pool


class Tee:
    """Duplicate stdout or stderr into a file (``log_dir/<host>_stdout.txt``)."""

    def __init__(self, path, err=False):
        self.file = open(path, "w")
        self.err = err
        self.stream = sys.stderr if err else sys.stdout
        if err:
            sys.stderr = self
        else:
            sys.stdout = self

    def close(self):
        if self.err:
            sys.stderr = self.stream
        else:
            sys.stdout = self.stream
        self.file.close()

    def write(self, data):
        try:
            self.file.write(data)
        except OSError:
            pass
        try:
            self.stream.write(data)
        except OSError:
            pass

    def flush(self):
        for s in (self.file, self.stream):
            try:
                s.flush()
            except OSError:
                pass


class NeoXArgs:
    """All configuration of one run; attribute access by key name (``args.hidden_size``)."""

    @staticmethod
    def known_keys():
        """Every declared argument name (the schema table)."""
        return list(FIELDS.keys())

    def __init__(self, **kwargs):
        unknown = [k for k in kwargs if k not in FIELDS]
        if unknown:
            raise TypeError(f"NeoXArgs got unexpected configuration key(s): {sorted(unknown)}")
        for name, f in FIELDS.items():
            object.__setattr__(self, name, copy.deepcopy(f.default))
        for k, v in kwargs.items():
            object.__setattr__(self, k, v)
        if self.git_hash is None:
            self.git_hash = git_commit_hash()
        # transient objects attached at run time (never serialised)
        self.tokenizer = None
        self.tensorboard_writer = None
        self.adlr_autoresume_object = None
        self.enable_logging()
        self.calculate_derived()
        if not self.validate_types():
            raise ValueError("NeoXArgs: a value has the wrong type")
        if not self.validate_values():
            raise ValueError("NeoXArgs: inconsistent values")

    # ------------------------------------------------------------------ construction
    @classmethod
    def from_ymls(cls, paths_to_yml_files, overwrite_values=None):
        config, config_files = {}, {}
        for path in paths_to_yml_files:
            with open(path) as fh:
                text = fh.read()
            conf = yaml.load(text, Loader=yaml.FullLoader) or {}
            for key, value in conf.items():
                key = key.replace("-", "_")
                if key in config:
                    raise ValueError(f"config file {path} repeats key '{key}' of an earlier file")
                config[key] = value
            base = os.path.basename(path)
            if base in config_files:
                raise AssertionError(f"two config files are both called {base}; names must be unique because "
                                     "they are saved side by side with each checkpoint")
            config_files[base] = text
        config["config_files"] = config_files
        if overwrite_values:
            config.update(overwrite_values)
        return cls(**config)

    @classmethod
    def from_dict(cls, args_dict):
        return cls(**args_dict)

    @classmethod
    def consume_deepy_args(cls, input_args=None):
        """Parse the launcher command line: ``deepy.py user_script [-d confdir] cfg1 cfg2 ...``."""
        p = argparse.ArgumentParser(description="neox-b200 launcher", allow_abbrev=False)
        p.add_argument("user_script", type=str, help="script to launch (train.py, generate.py, eval.py)")
        p.add_argument("--conf_dir", "-d", type=str, default=None, help="directory prefixed to every config path")
        p.add_argument("conf_file", type=str, nargs="+", help="YAML config file(s), merged")
        p.add_argument("--wandb_group", type=str, default=None)
        p.add_argument("--wandb_run_name", type=str, default=None)
        p.add_argument("--wandb_team", type=str, default=None)
        p.add_argument("--eval_tasks", type=str, nargs="+", default=None)
        p.add_argument("--iteration", type=int, default=None, help="checkpoint iteration for eval/generate")
        p.add_argument("--eval_results_prefix", type=str, default=None)
        p.add_argument("-H", "--hostfile", type=str)
        p.add_argument("-i", "--sample_input_file", type=str, default=None)
        p.add_argument("-o", "--sample_output_file", type=str, default=None)
        p.add_argument("--autotuning", type=str, default=None, choices=("tune", "run"))
        ns = p.parse_args(input_args)
        assert os.path.exists(ns.user_script), f"User script could not be found: {ns.user_script}"
        files = ns.conf_file
        if ns.conf_dir:
            files = [os.path.join(ns.conf_dir, f) for f in files]
        files = [f if f.endswith((".yml", ".json")) else f + ".yml" for f in files]
        overwrite = {}
        for k, v in vars(ns).items():
            if v is None or k in ("conf_dir", "conf_file"):
                continue
            overwrite["autotuning_run" if k == "autotuning" else k] = v
        args = cls.from_ymls(files, overwrite_values=overwrite)
        if args.use_wandb:
            import uuid
            suffix = uuid.uuid4().hex[:8]
            args.wandb_group = suffix if args.wandb_group is None else f"{args.wandb_group}_{suffix}"
        args.print()
        return args

    @classmethod
    def consume_neox_args(cls, overwrite_values=None, input_args=None):
        """Rebuild the args inside a worker from ``--megatron_config <urlsafe-b64 JSON>``."""
        p = argparse.ArgumentParser(allow_abbrev=False)
        p.add_argument("--megatron_config", type=str, default=None)
        p.add_argument("--deepspeed_config", type=str, default=None)
        ns, _ = p.parse_known_args(input_args)
        if ns.megatron_config is None:
            raise ValueError("worker started without --megatron_config; launch through deepy.py")
        cfg = json.loads(base64.urlsafe_b64decode(ns.megatron_config).decode("utf-8"))
        if ns.deepspeed_config is not None:
            try:
                ds = json.loads(base64.urlsafe_b64decode(ns.deepspeed_config).decode("utf-8"))
                overwrite_values = dict(overwrite_values or {})
                for key in AUTOTUNING_ARGS:
                    if key in ds and cfg.get("autotuning_run") is not None:
                        overwrite_values[key] = ds[key]
            except Exception:
                pass
        if overwrite_values:
            cfg.update(overwrite_values)
        return cls.from_dict(cfg)

    # ------------------------------------------------------------------ serialisation
    def _values(self, keys, only_non_defaults=False):
        out = {}
        for k in keys:
            v = getattr(self, k)
            if only_non_defaults and v == FIELDS[k].default:
                continue
            out[k] = v
        return out

    @property
    def all_config(self) -> dict:
        return self._values(FIELDS.keys())

    @property
    def megatron_config(self) -> dict:
        return self._values(k for k, f in FIELDS.items() if f.group not in ("engine", "runner"))

    @property
    def deepspeed_runner(self) -> dict:
        return self._values(RUNNER_KEYS)

    @property
    def deepspeed_config(self) -> dict:
        """Engine-level configuration (batch sizes, precision blocks, ZeRO, optimizer ...)."""
        cfg = self._values((k for k in ENGINE_KEYS if k != "deepspeed_extra_args"), only_non_defaults=True)
        if self.deepspeed_extra_args:
            non_default = self._values(FIELDS.keys(), only_non_defaults=True)
            for k, v in self.deepspeed_extra_args.items():
                if k in non_default and k != "bf16":
                    raise ValueError(f"key {k} is given both at top level and inside deepspeed_extra_args")
                cfg[k] = v
        return cfg

    @property
    def params_dtype(self):
        return {"fp16": torch.half, "bfloat16": torch.bfloat16}.get(self.precision, torch.float)

    @staticmethod
    def _cli(k, v):
        if isinstance(v, bool):
            return [f"--{k}"] if v else []
        return [] if v is None else [f"--{k}", str(v)]

    def get_deepspeed_main_args(self):
        """argv handed to the process launcher: runner flags, the user script, then the two blobs."""
        argv = []
        if self.autotuning_run is not None:
            argv += self._cli("autotuning", self.autotuning_run)
        for key in RUNNER_KEYS:
            if key == "autotuning_run":
                continue
            val = getattr(self, key)
            if key == "force_multi" and (self.deepspeed_slurm or self.deepspeed_mpi):
                val = True
            if key in ("comment", "account") and not self.deepspeed_slurm:
                continue
            if val != FIELDS[key].default:
                argv += self._cli(key, val)
        if "DLTS_HOSTFILE" in os.environ:
            argv += self._cli("hostfile", os.environ["DLTS_HOSTFILE"])
        if "MASTER_ADDR" in os.environ:
            argv += self._cli("master_addr", os.environ["MASTER_ADDR"])
        if ("--include" in argv or "--exclude" in argv) and "--num_gpus" in argv:
            i = argv.index("--num_gpus")
            del argv[i:i + 2]
        argv.append(self.user_script)
        self.configure_distributed_args()
        enc = lambda d: base64.urlsafe_b64encode(json.dumps(d).encode("utf-8")).decode("utf-8")
        argv += ["--deepspeed_config", enc(self.deepspeed_config)]
        argv += ["--megatron_config", enc(self._values(FIELDS.keys(), only_non_defaults=True))]
        return argv

    def save_yml(self, path):
        with open(path, "w") as fh:
            yaml.safe_dump(self._values(FIELDS.keys(), only_non_defaults=True), fh)

    # ------------------------------------------------------------------ mutation helpers
    def update_value(self, key, value):
        if key not in FIELDS:
            raise ValueError(f"NeoXArgs.update_value(): unknown key '{key}'")
        setattr(self, key, value)

    def update_values(self, d):
        for k, v in d.items():
            self.update_value(k, v)

    def build_tokenizer(self):
        from ..tokenizer import build_tokenizer
        self.tokenizer = build_tokenizer(self)

    def initialize_tensorboard_writer(self):
        if self.tensorboard_dir and self.rank == 0:
            try:
                from torch.utils.tensorboard import SummaryWriter
                self.tensorboard_writer = SummaryWriter(log_dir=self.tensorboard_dir)
            except (ModuleNotFoundError, ImportError):
                print("tensorboard is not installed; continuing without a tensorboard writer", flush=True)

    def initialize_comet(self):
        if self.use_comet and self.rank == 0:
            try:
                import comet_ml
                self.comet_experiment = comet_ml.Experiment(workspace=self.comet_workspace,
                                                            project_name=self.comet_project)
            except ModuleNotFoundError:
                print("comet_ml is not installed; continuing without Comet logging", flush=True)
                return
            exp = self.comet_experiment
            if hasattr(exp, "log_parameters"):
                exp.log_parameters(self._values(FIELDS.keys(), only_non_defaults=True))
            if self.comet_experiment_name:
                exp.set_name(self.comet_experiment_name)
            if self.comet_tags:
                exp.add_tags(self.comet_tags)
            if self.comet_others:
                exp.log_others(self.comet_others)

    # ------------------------------------------------------------------ logging
    def enable_logging(self):
        if self.log_dir:
            os.makedirs(self.log_dir, exist_ok=True)
            prefix = os.path.join(self.log_dir, gethostname())
            Tee(prefix + "_stdout.txt", err=False)
            Tee(prefix + "_stderr.txt", err=True)

    def print(self):
        if self.rank not in (0, None):
            return
        print("-------------------- arguments --------------------", flush=True)
        rows = []
        for k in FIELDS:
            v = getattr(self, k)
            tag = "default" if v == FIELDS[k].default else "updated"
            left = f"  {k} {'.' * max(1, 32 - len(k))} {v}"
            rows.append((tag, left + "." * max(1, 64 - len(left)) + tag))
        for _, line in sorted(rows, key=lambda r: (r[0] != "updated", r[1].lower())):
            print(line, flush=True)
        print("---------------- end of arguments ----------------", flush=True)

    # ------------------------------------------------------------------ distributed env
    def configure_distributed_args(self):
        if self.deepspeed_slurm:
            os.environ["LOCAL_RANK"] = os.environ["SLURM_LOCALID"]
            os.environ["RANK"] = os.environ["SLURM_PROCID"]
            os.environ["WORLD_SIZE"] = os.environ.get("SLURM_NTASKS") or str(
                int(os.environ["SLURM_NNODES"]) * int(os.environ["SLURM_NTASKS_PER_NODE"]))
        if self.deepspeed_mpi and "OMPI_COMM_WORLD_RANK" in os.environ:
            os.environ["RANK"] = os.environ["OMPI_COMM_WORLD_RANK"]
            os.environ["LOCAL_RANK"] = os.environ.get("OMPI_COMM_WORLD_LOCAL_RANK", "0")
            os.environ["WORLD_SIZE"] = os.environ["OMPI_COMM_WORLD_SIZE"]
        self.local_rank = int(os.getenv("LOCAL_RANK", "0"))
        self.rank = int(os.getenv("RANK", "0"))
        self.world_size = int(os.getenv("WORLD_SIZE", "1"))
        if self.rank == 0:
            print(f"NeoXArgs.configure_distributed_args() using world size: {self.world_size} and "
                  f"model-parallel size: {self.model_parallel_size}", flush=True)

    # ------------------------------------------------------------------ derived values
    @staticmethod
    def calculate_batch_parameters(dp_world_size, train_batch=None, micro_batch=None, grad_acc=None):
        """Fill in whichever of (train_batch, micro_batch, grad_acc) is missing."""
        dp = int(dp_world_size)
        if train_batch is not None and micro_batch is not None and grad_acc is not None:
            pass
        elif train_batch is not None and micro_batch is not None:
            grad_acc = (train_batch // micro_batch) // dp
        elif train_batch is not None and grad_acc is not None:
            micro_batch = (train_batch // dp) // grad_acc
        elif micro_batch is not None and grad_acc is not None:
            train_batch = micro_batch * grad_acc * dp
        elif train_batch is not None:
            grad_acc, micro_batch = 1, train_batch // dp
        elif micro_batch is not None:
            train_batch, grad_acc = micro_batch * dp, 1
        else:
            raise AssertionError("Either train_batch_size or train_micro_batch_size_per_gpu needs to be provided")
        return int(train_batch), int(micro_batch), int(grad_acc)

    @staticmethod
    def check_batch_parameters(dp_world_size, train_batch, micro_batch, grad_acc):
        assert train_batch > 0, f"Train batch size: {train_batch} has to be greater than 0"
        assert micro_batch > 0, f"Micro batch size per gpu: {micro_batch} has to be greater than 0"
        assert grad_acc > 0, f"Gradient accumulation steps: {grad_acc} has to be greater than 0"
        assert train_batch == micro_batch * grad_acc * dp_world_size, (
            "train_batch_size must equal micro_batch_per_gpu * gradient_acc_step * data-parallel world size: "
            f"{train_batch} != {micro_batch} * {grad_acc} * {dp_world_size}")

    def _count_gpus(self):
        n = self.global_num_gpus
        if n is not None:
            return n
        hostfile = self.hostfile or (DLTS_HOSTFILE if os.path.exists(DLTS_HOSTFILE) else None)
        if hostfile is not None:
            pool = resource_pool(hostfile, self.include or "", self.exclude or "")
            if self.num_nodes is not None and self.num_nodes > 0:
                pool = dict(list(pool.items())[: self.num_nodes])
            n = sum(len(v) for v in pool.values())
            if self.num_gpus is not None and self.num_gpus > 0:
                n = self.num_gpus * len(pool)
        elif os.environ.get("WORLD_SIZE") and "RANK" in os.environ:
            n = int(os.environ["WORLD_SIZE"])
        else:
            n = torch.cuda.device_count()
            if self.num_gpus is not None and self.num_gpus > 0:
                n = self.num_gpus
        return n

    def calculate_derived(self):
        gpus = self._count_gpus()
        self.global_num_gpus = gpus
        pp = max(self.pipe_parallel_size, 1)
        mp = max(self.model_parallel_size, 1)
        self.model_parallel_size = mp
        dp = (gpus / pp) / mp
        if dp % 1 != 0:
            raise AssertionError(f"(global_num_gpus / pp_size) / mp_size [({gpus} / {pp}) / {mp}] must be a whole number")
        if self.elasticity and self.elasticity.get("enabled", False):
            # the elastic batch replaces the configured triple (an explicit one must agree with it unless told so)
            from .elasticity import compute_elastic_config
            e_batch, _, e_micro = compute_elastic_config(self.elasticity, world_size=int(dp))
            given = (self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps)
            if not self.elasticity.get("ignore_non_elastic_batch_info", False) and any(v is not None for v in given):
                if self.train_batch_size not in (None, e_batch):
                    raise AssertionError(
                        f"train_batch_size {self.train_batch_size} disagrees with the elastic batch size {e_batch}; "
                        "remove it or set elasticity.ignore_non_elastic_batch_info")
            self.train_batch_size, self.train_micro_batch_size_per_gpu = e_batch, e_micro
            self.gradient_accumulation_steps = e_batch // (e_micro * int(dp))
        tb, mb, ga = self.calculate_batch_parameters(dp, self.train_batch_size, self.train_micro_batch_size_per_gpu,
                                                     self.gradient_accumulation_steps)
        self.check_batch_parameters(dp, tb, mb, ga)
        self.train_batch_size, self.train_micro_batch_size_per_gpu, self.gradient_accumulation_steps = tb, mb, ga
        self.batch_size = mb
        self.clip_grad = self.gradient_clipping

        # precision
        if self.fp16 and self.fp16.get("enabled", False):
            assert self.precision in (None, "fp16"), "fp16 block is enabled but precision says otherwise"
            self.precision = "fp16"
        if self.bf16 and self.bf16.get("enabled", False):
            assert self.precision in (None, "bfloat16"), "bf16 block is enabled but precision says otherwise"
            self.precision = "bfloat16"
        if self.zero_optimization is None:
            self.zero_optimization = copy.deepcopy(ZERO_DEFAULTS)
        if self.precision == "fp16":
            block = copy.deepcopy(self.fp16) if isinstance(self.fp16, dict) and self.fp16 else {"type": "fp16"}
            block["enabled"] = True
            self.fp16 = block
        elif self.precision == "bfloat16":
            if not self.bf16:
                extra = copy.deepcopy(self.deepspeed_extra_args) or {}
                extra["bf16"] = {"enabled": True}
                self.deepspeed_extra_args = extra
        else:
            self.precision = "fp32"

        # ZeRO
        stage = self.zero_optimization["stage"]
        if stage in (0, 1, 2, 3):
            z = self.zero_optimization
            self.zero_stage = stage
            self.zero_reduce_scatter = z.get("reduce_scatter", ZERO_DEFAULTS["reduce_scatter"])
            self.zero_contiguous_gradients = z.get("contiguous_gradients", ZERO_DEFAULTS["contiguous_gradients"])
            self.zero_reduce_bucket_size = z.get("reduce_bucket_size", ZERO_DEFAULTS["reduce_bucket_size"])
            self.zero_allgather_bucket_size = z.get("allgather_bucket_size", ZERO_DEFAULTS["allgather_bucket_size"])
        else:
            assert self.autotuning is not None, f"Zero Stage must be an integer unless you are doing autotuning, not {stage}"

        # optimizer
        opt = self.optimizer or {"type": OPT_DEFAULT, "params": OPT_PARAMS_DEFAULTS}
        self.optimizer_type = opt.get("type", OPT_DEFAULT)
        self.lr = opt.get("params", {}).get("lr", OPT_PARAMS_DEFAULTS["lr"])
        if isinstance(self.lr, str):            # YAML 1.1 reads "1e-4" (no dot) as a string
            self.lr = float(self.lr)
        if self.optimizer_type.lower() == "onebitadam":
            assert self.train_iters is not None, "OneBitAdam requires train_iters to be specified"
            self.scheduler = {"type": "WarmupDecayLR",
                              "params": {"warmup_min_lr": 0, "warmup_max_lr": self.lr,
                                         "warmup_num_steps": int(self.train_iters * self.warmup),
                                         "total_num_steps": self.lr_decay_iters or self.train_iters}}
        self.dynamic_loss_scale = self.loss_scale is None

        # pipeline / MoE exclusions
        self.is_pipe_parallel = self.pipe_parallel_size >= 1
        if self.moe_num_experts > 1:
            assert not self.is_pipe_parallel, "MoE not supported with pipeline parallelism"
            assert self.zero_optimization["stage"] != 3, "MoE not compatible with zero3"
            assert self.sequence_parallel is False, "MoE not compatible with Sequence Parallel"

        # attention pattern
        if self.num_layers is not None:
            cfg = self.attention_config if self.attention_config is not None else [[["global"], self.num_layers]]
            self.attention_config = expand_attention_types(cfg, self.num_layers)
            assert len(self.attention_config) == self.num_layers, "Length of attention config list must equal num_layers"
            for kind in self.attention_config:
                assert kind in ATTENTION_TYPE_CHOICES, f"Attention type {kind} not recognized"
            kinds = set(self.attention_config)
            if kinds & {"gmlp", "amlp"}:
                assert not self.partition_activations, "GMLP Blocks are not compatible with partition activations"
            if "mamba" in kinds and isinstance(self.zero_stage, int):
                assert self.zero_stage <= 2, "Zero stage 3 not compatible with Mamba"
            if "rwkv" in kinds:
                assert self.model_parallel_size == 1, "RWKV not currently compatible with model parallelism"
                if isinstance(self.zero_stage, int):
                    assert self.zero_stage <= 2, "Zero stage 3 not compatible with RWKV"
        if self.sparsity_config is None:
            self.sparsity_config = {}

        # grouped-query attention
        if self.num_kv_heads is not None and self.num_attention_heads is not None:
            assert self.num_attention_heads % self.num_kv_heads == 0, \
                "num_kv_heads must evenly divide num_attention_heads and be no greater than it"
            if self.num_kv_heads < self.num_attention_heads:
                assert not self.sparsity_config, "Sparse attention not compatible with GQA or MQA"
                assert all(k in ("flash", "global") for k in (self.attention_config or [])), \
                    "GQA / MQA currently only compatible with Flash or standard global/sliding window Attention"
                assert self.num_kv_heads % self.model_parallel_size == 0, \
                    "Number of KV heads must be at least model_parallel_size for now!"

        # dataset weights default to uniform
        for split in ("train", "valid", "test"):
            paths = getattr(self, f"{split}_data_paths") or getattr(self, f"pos_{split}_data_paths")
            if paths and getattr(self, f"{split}_data_weights") is None:
                setattr(self, f"{split}_data_weights", [1.0] * len(paths))
        if self.train_label_data_paths:
            assert self.train_data_paths and not self.data_path, \
                "Must use `train_label_data_paths` with `train_data_paths`, not `data_path`"
        if self.text_gen_type is None:
            self.text_gen_type = "input-file" if self.sample_input_file else "unconditional"

    # ------------------------------------------------------------------ validation
    def validate_types(self) -> bool:
        for name, f in FIELDS.items():
            v = getattr(self, name)
            if not f.accepts(v):
                logging.error(f"NeoXArgs.validate_types() {name}: expected {f.type_str()}, got "
                              f"{type(v).__name__} ({v!r})")
                return False
        for name in ("optimizer", "scheduler"):
            block = getattr(self, name)
            if isinstance(block, dict):
                if "type" not in block:
                    logging.error(f"NeoXArgs.validate_types() {name}: key 'type' must be defined")
                    return False
                if not isinstance(block["type"], str) or not isinstance(block.get("params", {}), dict):
                    logging.error(f"NeoXArgs.validate_types() {name}: 'type' must be str and 'params' a dict")
                    return False
        for name in ("fp16", "amp", "flops_profiler"):
            block = getattr(self, name)
            if isinstance(block, dict):
                if "enabled" not in block:
                    logging.error(f"NeoXArgs.validate_types() {name}: key 'enabled' must be defined")
                    return False
                if not isinstance(block["enabled"], bool):
                    logging.error(f"NeoXArgs.validate_types() {name}: 'enabled' must be a bool")
                    return False
        return True

    def validate_values(self) -> bool:
        if not self.deepspeed:
            return False

        def fail(msg):
            logging.error("NeoXArgs.validate_values() " + msg)
            raise ValueError("NeoXArgs.validate_values() " + msg)

        if self.lr is None:
            fail("lr is None")
        for req in ("num_layers", "hidden_size", "num_attention_heads", "max_position_embeddings"):
            if getattr(self, req) is None:
                fail(f"{req} is None.")
        if self.hidden_size % self.num_attention_heads != 0 and "mamba" not in self.attention_config:
            fail("hidden_size must be divisible by num_attention_heads")
        if self.seq_length is not None and self.max_position_embeddings < self.seq_length:
            fail("max_position_embeddings must be bigger or equal seq_length")
        if self.min_lr > self.lr:
            fail("min_lr must be smaller or equal lr")
        if self.save is not None and self.checkpoint_factor is None and self.extra_save_iters is None:
            fail("checkpoint_factor or extra_save_iters must be defined if save is defined")
        if self.num_unique_layers is not None and self.num_layers is not None:
            if self.num_unique_layers > self.num_layers:
                fail("num-unique-layers must be smaller or equal num_layers")
            if self.num_layers % self.num_unique_layers != 0:
                fail("num-layers should be divisible by num-unique-layers")
        if self.fp16_lm_cross_entropy and self.precision != "fp16":
            fail("lm cross entropy in fp16 only support in fp16 mode.")
        separate = [p is not None for p in (self.train_data_paths, self.valid_data_paths, self.test_data_paths)]
        if all(separate):
            assert self.data_path is None, "Please provide *either* `data_path` or `train/valid/test_data_path`"
        assert any(separate) == all(separate), (
            "One or more of train/valid/test data_path are not provided: "
            f"train {self.train_data_paths}, valid {self.valid_data_paths}, test {self.test_data_paths}")
        for split in ("train", "valid", "test"):
            paths, weights = getattr(self, f"{split}_data_paths"), getattr(self, f"{split}_data_weights")
            if paths is not None and weights is not None:
                assert len(paths) == len(weights), f"{split}_data_paths and {split}_data_weights differ in length"
        if self.sequence_parallel and self.model_parallel_size > 1 and self.seq_length is not None:
            if self.seq_length % self.model_parallel_size != 0:
                fail("seq_length must be divisible by model_parallel_size when sequence_parallel is on")
        return True

    # convenience used throughout the code base -------------------------------------------------
    @property
    def dp_world_size(self) -> int:
        return int(self.global_num_gpus // (max(self.pipe_parallel_size, 1) * self.model_parallel_size))

    def __repr__(self):
        return f"NeoXArgs({self._values(FIELDS.keys(), only_non_defaults=True)})"
