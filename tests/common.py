"""Shared helpers for the test-suite: tiny model configs and a multi-process (gloo) launcher."""
import os
import socket
import sys
import tempfile
import traceback

import torch
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

BASE_CONFIG = {
    "num_layers": 2, "hidden_size": 64, "num_attention_heads": 4, "seq_length": 32, "max_position_embeddings": 32,
    "pos_emb": "rotary", "rotary_pct": 0.25, "no_weight_tying": True, "gpt_j_residual": True,
    "output_layer_parallelism": "column", "norm": "layernorm",
    "init_method": "small_init", "output_layer_init_method": "wang_init",
    "optimizer": {"type": "Adam", "params": {"lr": 1e-3, "betas": [0.9, 0.95], "eps": 1e-8}},
    "zero_optimization": {"stage": 0}, "train_micro_batch_size_per_gpu": 2, "gradient_accumulation_steps": 1,
    "train_iters": 20, "lr_decay_iters": 20, "lr_decay_style": "cosine", "warmup": 0.1, "min_lr": 1e-4,
    "weight_decay": 0.01, "gradient_clipping": 1.0, "hidden_dropout": 0.0, "attention_dropout": 0.0,
    "precision": "fp32", "data_path": "synthetic", "tokenizer_type": "CharLevelTokenizer",
    "make_vocab_size_divisible_by": 64, "log_interval": 1000, "eval_interval": 100000, "eval_iters": 1,
    "num_workers": 0, "seed": 1234, "distributed_backend": "gloo", "global_num_gpus": 1,
    "attention_config": [[["global"], "all"]], "checkpoint_factor": 1000,
}


def make_args(**overrides):
    from gpt_neox_b200.config import NeoXArgs
    cfg = dict(BASE_CONFIG)
    cfg.update(overrides)
    args = NeoXArgs.from_dict(cfg)
    args.build_tokenizer()
    return args


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, fn_args, errq):
    os.environ.update(RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE=str(world), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port))
    sys.path.insert(0, ROOT)
    try:
        # the models are tiny and several ranks (often several jobs) share the host: a full-width intra-op thread
        # pool per rank only makes them fight for the cores
        torch.set_num_threads(2)
        torch.manual_seed(0)
        fn(rank, world, *fn_args)
    except Exception:
        errq.put((rank, traceback.format_exc()))
    finally:
        import torch.distributed as dist
        if dist.is_initialized():
            try:
                dist.destroy_process_group()
            except Exception:
                pass


def run_distributed(fn, world_size, *fn_args, timeout=300):
    """Run ``fn(rank, world, *args)`` in ``world_size`` spawned processes (gloo on CPU)."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world_size, port, fn, fn_args, errq)) for r in range(world_size)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout)
    hung = [p for p in procs if p.is_alive()]
    for p in hung:
        p.terminate()
    errs = []
    while not errq.empty():
        errs.append(errq.get())
    assert not hung, f"{len(hung)} rank(s) did not finish within {timeout}s"
    assert not errs, "\n".join(f"[rank {r}]\n{tb}" for r, tb in errs)
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]


def run_distributed_many(*calls, timeout=300):
    """Several independent ``run_distributed(fn, world, *args)`` jobs side by side (each with its own processes and
    port): the baseline and the variant of a comparison do not have to wait for one another."""
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=len(calls)) as pool:
        futures = [pool.submit(run_distributed, *c, timeout=timeout) for c in calls]
        for f in futures:
            f.result()

