"""Tensor-parallel parity of whole-model training on GPUs (launched by torchrun from test_fused_comm_gpu.py).

Trains the same small GPT-NeoX model (parallel residual, rotary, flash attention, activation checkpointing, bf16) for
ten steps on identical data with the weights drawn on the host (``use_cpu_initialization``: the full matrix is drawn
once and sliced, so every tensor-parallel degree starts from the same parameters), with tensor parallel degree =
the number of ranks.  With more than one rank the run is done twice: through the fused compute+collective kernels
and through the NCCL mappings.  The per-step losses are written to ``$TP_PARITY_OUT`` as JSON by rank 0; the test
compares the files of the 1-, 2- and 4-rank runs.
"""
import json
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def run(fused, sp):
    from common import make_args
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.parallel import fused_comm, mpu
    from gpt_neox_b200.training import setup_model_and_optimizer, train_step
    from gpt_neox_b200.utils import Timers
    world = int(os.environ["WORLD_SIZE"])
    os.environ["NEOX_FUSED_TP_COMM"] = "1" if fused else "0"
    args = make_args(hidden_size=1024, num_attention_heads=8, num_layers=4, seq_length=512, max_position_embeddings=512,
                     precision="bfloat16", global_num_gpus=world, model_parallel_size=world, distributed_backend="nccl",
                     sequence_parallel=sp and world > 1, zero_optimization={"stage": 1},
                     train_micro_batch_size_per_gpu=2, gradient_accumulation_steps=2, checkpoint_activations=True,
                     attention_config=[[["flash"], "all"]], use_cpu_initialization=True, train_iters=100,
                     lr_decay_iters=100, warmup=0.0, seed=1234,
                     optimizer={"type": "Adam", "params": {"lr": 3e-4, "betas": [0.9, 0.95], "eps": 1e-8}})
    args.configure_distributed_args()
    initialize_megatron(args)
    torch.manual_seed(1234)
    model, opt, sched, _ = setup_model_and_optimizer(args)
    g = torch.Generator().manual_seed(11)
    batches = [{"text": torch.randint(0, args.padded_vocab_size, (2, 513), generator=g)} for _ in range(4)]

    def it():
        i = 0
        while True:
            yield batches[i % 4]
            i += 1
    data = it()
    losses = []
    for _ in range(10):
        d, _ = train_step(args, Timers(), data, model, opt, sched)
        losses.append(float(d["lm_loss"]))
    from gpt_neox_b200.ops import native
    status = native.read_status()
    fused_comm.reset()
    mpu.destroy_model_parallel()
    return losses, status


def main():
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    world = int(os.environ["WORLD_SIZE"])
    out = {}
    modes = [("nccl", False, False)] if world == 1 else [("fused", True, False), ("nccl", False, False),
                                                         ("fused_sp", True, True)]
    bad = 0
    for name, fused, sp in modes:
        losses, status = run(fused, sp)
        out[name] = losses
        bad |= int(status != 0)
    if dist.get_rank() == 0:
        with open(os.environ["TP_PARITY_OUT"], "w") as fh:
            json.dump(out, fh)
        print(("TP_PARITY_DONE" if not bad else "TP_PARITY_STATUS_NONZERO"), out, flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(bad)


if __name__ == "__main__":
    main()
