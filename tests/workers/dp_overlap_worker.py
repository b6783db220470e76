"""2-GPU data-parallel ZeRO-1 training with and without overlapped communication (launched by torchrun).

Trains the same tiny bf16 model twice from the same seed -- gradient reduce-scatter at the optimizer step vs.
bucketed reduce-scatter started from backward hooks on a side stream plus asynchronous parameter all-gather --
and checks that the losses agree and that buckets were really reduced early; then both once more with the gradient
reduce-scatter and the parameter all-gather done by the peer-memory kernels instead of NCCL (``NEOX_ZERO_PEER=1``):
same losses, no bounded wait expired; and once each with ZeRO stage 2 (gradient partitioning) and stage 3 (parameter partitioning).  Prints ``DP_OVERLAP_OK``
on rank 0.
"""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def run(overlap, stage=1):
    from common import make_args
    from gpt_neox_b200.parallel import mpu
    from gpt_neox_b200.training import setup_model_and_optimizer, train_step
    from gpt_neox_b200.utils import Timers
    world = int(os.environ["WORLD_SIZE"])
    zero = {"stage": stage, "overlap_comm": True, "reduce_bucket_size": 300000} if overlap else {"stage": stage}
    args = make_args(hidden_size=256, num_attention_heads=4, num_layers=4, seq_length=128, max_position_embeddings=128,
                     precision="bfloat16", global_num_gpus=world, distributed_backend="nccl", zero_optimization=zero,
                     train_micro_batch_size_per_gpu=4, gradient_accumulation_steps=2,
                     attention_config=[[["flash"], "all"]])
    from gpt_neox_b200.initialize import initialize_megatron
    args.configure_distributed_args()
    initialize_megatron(args)
    torch.manual_seed(1234)
    model, opt, sched, _ = setup_model_and_optimizer(args)
    g = torch.Generator().manual_seed(7 + mpu.get_data_parallel_rank())
    batches = [{"text": torch.randint(0, args.padded_vocab_size, (4, 129), generator=g)} for _ in range(4)]

    def it():
        i = 0
        while True:
            yield batches[i % 4]
            i += 1
    data = it()
    losses = []
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for i in range(8):
        if i == 3:
            torch.cuda.synchronize()
            t0.record()
        d, _ = train_step(args, Timers(), data, model, opt, sched)
        losses.append(float(d["lm_loss"]))
    t1.record()
    torch.cuda.synchronize()
    run.ms = t0.elapsed_time(t1) / 5
    run.peer = all(getattr(b, "peer", False) for b in opt.buckets)
    return losses, getattr(opt, "overlapped_reductions", 0), len(opt.buckets)


def main():
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    os.environ["NEOX_ZERO_PEER"] = "0"
    plain, _, nb0 = run(False)
    over, early, nb1 = run(True)
    ms_over = run.ms
    ok = all(abs(a - b) < 2e-2 for a, b in zip(plain, over)) and early > 0 and nb1 > nb0 and not run.peer
    if not ok:
        print(f"[rank {dist.get_rank()}] plain {plain} overlap {over} early {early} buckets {nb0}->{nb1}", flush=True)
    # the same two runs with the data-parallel traffic on the peer-memory kernels
    from gpt_neox_b200.ops import native
    os.environ["NEOX_ZERO_PEER"] = "1"
    peer_plain, _, _ = run(False)
    used = run.peer
    peer_over, early_p, _ = run(True)
    used = used and run.peer
    ms_peer = run.ms
    os.environ["NEOX_ZERO_PEER"] = "0"
    status = native.read_status()
    ok_peer = (used and status == 0 and early_p > 0 and all(abs(a - b) < 2e-2 for a, b in zip(plain, peer_plain))
               and all(abs(a - b) < 2e-2 for a, b in zip(plain, peer_over)))
    if not ok_peer:
        print(f"[rank {dist.get_rank()}] peer traffic: used {used} status {status} early {early_p} plain {plain} "
              f"peer {peer_plain} peer+overlap {peer_over}", flush=True)
    elif dist.get_rank() == 0:
        print(f"ZERO_PEER_OK ms/step overlapped: nccl {ms_over:.2f} peer {ms_peer:.2f}", flush=True)
    ok = ok and ok_peer
    # ZeRO stage 2 (transient full-size gradient buffers, one reduce-scatter per micro-batch), with the reductions
    # on the side stream: same losses, and no full-size gradient buffer left between steps
    z2, _, _ = run(True, stage=2)
    ok_z2 = all(abs(a - b) < 2e-2 for a, b in zip(plain, z2))
    if not ok_z2:
        print(f"[rank {dist.get_rank()}] stage 2: plain {plain} stage2 {z2}", flush=True)
    elif dist.get_rank() == 0:
        print(f"ZERO2_OK ms/step {run.ms:.2f}", flush=True)
    ok = ok and ok_z2
    # ZeRO stage 3: parameters gathered per layer right before use, only shards held between steps
    z3, _, _ = run(True, stage=3)
    ok_z3 = all(abs(a - b) < 2e-2 for a, b in zip(plain, z3))
    if not ok_z3:
        print(f"[rank {dist.get_rank()}] stage 3: plain {plain} stage3 {z3}", flush=True)
    elif dist.get_rank() == 0:
        print(f"ZERO3_OK ms/step {run.ms:.2f}", flush=True)
    ok = ok and ok_z3
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if dist.get_rank() == 0 and flag.item() == 1:
        print("DP_OVERLAP_OK", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
