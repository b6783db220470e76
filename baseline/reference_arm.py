"""Reference arm of bench.py: times the stock reference training step on the same configuration.

What runs: the unmodified reference tree copied to ``baseline/_ref`` -- its NeoXArgs, ``initialize_megatron``,
``setup_model_and_optimizer`` (``get_model`` -> ``GPT2ModelPipe``, ``mpu`` Column/RowParallelLinear on cuBLAS + NCCL,
flash-attn, torch LayerNorm, vocab-parallel cross entropy) and ``train_step`` -- driven through those public
functions.  DeepSpeed, which the reference imports at module scope and which cannot be installed offline, is replaced
by the pure-PyTorch stand-in under ``baseline/ds_shim`` (engine only: bf16 parameters + fp32 master weights +
torch fused AdamW, NCCL gradient reduction, 1F1B for pipeline stages).  Nothing from ``gpt_neox_b200`` is imported
and none of its native libraries is loaded on this path.

The reference's fused softmax / rope kernels are JIT-built for sm_70..sm_90 only and cannot load on sm_100, so the
fusion flags that need them are off; with flash attention selected they are not on the step path anyway.
"""
import json
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SHIM = os.path.join(HERE, "ds_shim")


def ensure_reference_tree():
    """baseline/_ref is a plain copy of the reference tree (it is a script tree: pip cannot install it)."""
    if os.path.isdir(os.path.join(REF, "megatron")):
        return None
    src = os.environ.get("NEOX_REFERENCE_SRC", "")          # where a checkout of the reference can be copied from
    if src and os.path.isdir(os.path.join(src, "megatron")):
        try:
            shutil.copytree(src, REF, dirs_exist_ok=True)
            return None
        except Exception as exc:  # pragma: no cover
            return f"copying the reference tree to baseline/_ref failed ({type(exc).__name__}: {exc})"
    return "baseline/_ref is absent (set NEOX_REFERENCE_SRC to a checkout of the reference to have it copied)"


def flops_per_iteration(batch, seq, layers, hidden, vocab, c):
    """The reference's own count (megatron/logging.py:146-160): 24*c*B*s*L*h^2*(1 + s/6h + V/16Lh)."""
    return 24.0 * c * batch * seq * layers * hidden ** 2 * (1.0 + seq / (6.0 * hidden) + vocab / (16.0 * layers * hidden))


def run(a, cfg, vocab_size, depth_of, clock_sampler_cls, metric, model_desc):
    why = ensure_reference_tree()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    for k in [k for k in sys.modules if k == "gpt_neox_b200" or k.startswith("gpt_neox_b200.")]:
        raise RuntimeError("the reference arm must not share a process with gpt_neox_b200")
    sys.path.insert(0, REF)
    sys.path.insert(0, SHIM)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29511")
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("WORLD_SIZE", "1")

    import torch
    import torch.distributed as dist
    n = a.gpus
    world = int(os.environ["WORLD_SIZE"])
    assert world == n, f"--gpus {n} but WORLD_SIZE={world}"
    if not torch.cuda.is_available():
        print(json.dumps({"impl": "reference", "unavailable": "the reference asserts CUDA (megatron/initialize.py:42) and no GPU is visible"}))
        return 0

    cfg = dict(cfg)
    # kernels the reference can only JIT-build for sm_70..sm_90; not on the flash-attention step path
    cfg.update({"scaled_upper_triang_masked_softmax_fusion": False, "scaled_masked_softmax_fusion": False,
                "rope_fusion": False})
    cfg.pop("global_num_gpus", None)

    from megatron.neox_arguments import NeoXArgs
    from megatron.initialize import initialize_megatron
    from megatron import mpu
    from megatron.training import setup_model_and_optimizer, train_step
    from megatron.utils import Timers

    neox_args = NeoXArgs.from_dict(cfg)
    neox_args.configure_distributed_args()
    neox_args.build_tokenizer()
    neox_args.padded_vocab_size = vocab_size
    initialize_megatron(neox_args)
    rank = dist.get_rank()
    dev = torch.device("cuda", torch.cuda.current_device())
    model, optimizer, lr_scheduler, _ = setup_model_and_optimizer(neox_args, use_cache=False)
    timers = Timers(use_wandb=False, tensorboard_writer=None, comet_experiment=None)
    gas, mb, seq = neox_args.gradient_accumulation_steps, neox_args.train_micro_batch_size_per_gpu, neox_args.seq_length

    g = torch.Generator().manual_seed(1234 + mpu.get_data_parallel_rank())
    pool = max(gas, 8)
    host = [torch.randint(0, vocab_size, (mb, seq + 1), generator=g, dtype=torch.int64).pin_memory() for _ in range(pool)]
    on_dev = [t.to(dev) for t in host]
    # the reference reads data on tensor-parallel rank 0 of the first and last pipeline stage and broadcasts it
    reads = mpu.get_model_parallel_rank() == 0 and (
        not neox_args.is_pipe_parallel or mpu.get_pipe_parallel_rank() in (0, mpu.get_pipe_parallel_world_size() - 1))

    def stream(tensors):
        i = 0
        while True:
            yield {"text": tensors[i % len(tensors)]}
            i += 1

    def run_steps(k, it, read_loss):
        last = None
        for _ in range(k):
            d, _ = train_step(neox_args=neox_args, timers=timers, data_iterator=it if reads else None, model=model,
                              optimizer=optimizer, lr_scheduler=lr_scheduler)
            neox_args.iteration += 1
            if read_loss:
                last = float(d["lm_loss"])
        return last

    def timed(k, it, read_loss):
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        loss = run_steps(k, it, read_loss)
        e1.record()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ms = torch.tensor([e0.elapsed_time(e1)], device=dev)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms) / k, loss

    warm = max(a.warmup, 3)
    run_steps(warm, stream(on_dev), True)
    sampler = clock_sampler_cls(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    ms_dev, _ = timed(a.steps, stream(on_dev), False)
    ms_e2e, loss = (None, None) if a.skip_e2e else timed(a.steps, stream(host), True)
    clocks = sampler.stop() if rank == 0 else None

    tokens = neox_args.train_batch_size * seq
    depth = depth_of(neox_args.num_layers)
    fl = lambda c: flops_per_iteration(neox_args.train_batch_size, seq, neox_args.num_layers, neox_args.hidden_size,
                                       vocab_size, c) / (ms_dev / 1e3) / n / 1e12
    if rank == 0:
        tp = neox_args.model_parallel_size
        pp = neox_args.pipe_parallel_size
        out = {
            "impl": "reference", "metric": metric, "value": round(tokens / (ms_dev / 1e3) * depth, 1), "unit": "tokens/s",
            "n_gpus": n, "steps": a.steps, "warmup": warm, "ms_per_step": round(ms_dev, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init weights (small_init / wang_init)",
            "tflops_per_gpu": {"model_c3": round(fl(3), 1),
                               "hardware_c4": round(fl(4 if neox_args.checkpoint_activations else 3), 1)},
            "config": {"model": model_desc(neox_args.num_layers, neox_args.hidden_size),
                       "global_batch": neox_args.train_batch_size, "seq_len": seq, "micro_batch": mb, "grad_accum": gas,
                       "activation_checkpointing": bool(neox_args.checkpoint_activations),
                       "parallelism": f"tp{tp}" + (f"pp{pp}" if pp else "") + f"dp{world // (tp * max(pp, 1))}"
                                      + (" sp" if neox_args.sequence_parallel else "") + " zero1",
                       "l2": "inputs larger than L2 (no flush needed)"},
            "reference_path": "stock megatron/ model, mpu, flash-attn and train_step from baseline/_ref; DeepSpeed engine "
                              "replaced by the pure-PyTorch stand-in baseline/ds_shim; softmax/rope JIT fusions off "
                              "(sm_90-only build), flash attention on",
            "clocks": clocks,
            "e2e": None if ms_e2e is None else {"value": round(tokens / (ms_e2e / 1e3) * depth, 1), "unit": "tokens/s",
                                                "ms_per_step": round(ms_e2e, 2),
                                                "h2d_bytes_per_step": gas * mb * (seq + 1) * 8,
                                                "d2h_bytes_per_step": 4, "final_loss": loss},
            "tokens_per_sec_at_measured_depth": round(tokens / (ms_dev / 1e3), 1),
            "gpu_launches": 0,
            "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 1),
        }
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0
