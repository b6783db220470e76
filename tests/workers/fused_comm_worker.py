"""Multi-GPU worker for the fused tensor-parallel GEMM tests (launched by torchrun from test_fused_comm_gpu.py).

Every check compares a fused peer-memory op with the NCCL collective + fp32 matmul statement of the same math.
Prints ``FUSED_COMM_OK`` on rank 0 when all checks pass on all ranks.
"""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from gpt_neox_b200.ops import native  # noqa: E402
from gpt_neox_b200.parallel import fused_comm, mpu  # noqa: E402


def close(a, b, tol, what):
    a, b = a.float(), b.float()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item() + 1e-6
    ok = err <= tol * ref
    if not ok:
        print(f"[rank {dist.get_rank()}] MISMATCH {what}: max err {err:.4g} vs ref max {ref:.4g}", flush=True)
    return ok


def main():
    rank = int(os.environ["RANK"])
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    dist.init_process_group("nccl")
    mpu.initialize_model_parallel(world)
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = fused_comm.workspace()
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    ok = True
    rows, K, N = 256, 512, 768                     # per-rank rows; small enough for seconds, > 1 tile each way
    grp = mpu.get_model_parallel_group()

    def rnd(*shape, scale=1.0):
        return (torch.randn(*shape, device=dev, generator=g) * scale).to(torch.bfloat16)

    for it in range(5):                            # > 2 iterations: both buffer parities get reused
        # ---- all-gather -> GEMM: the shards arrive while the GEMM runs; K-major B, then MN-major B
        x = rnd(rows, K)
        w = rnd(N, K, scale=0.05)
        full = torch.empty(rows * world, K, device=dev, dtype=torch.bfloat16)
        dist.all_gather_into_tensor(full, x, group=grp)
        h = ws.begin_gather(x)
        y = ws.gemm(h.full, w, gather=h, bcast=True, dep="a")
        ok &= close(y, full.float() @ w.float().t(), 2e-2, f"ag_gemm it{it}")
        ok &= bool(torch.equal(h.full, full))
        w2 = rnd(K, N, scale=0.05)
        y2 = ws.gemm(h.full, w2, False, True, gather=h, dep="a")       # second reader of the same gathered buffer
        ok &= close(y2, full.float() @ w2.float(), 2e-2, f"ag_gemm(b_mn) it{it}")
        ws.release(h)
        # ---- wgrad with the gathered operand on the A side:  dW[K, N2] = full^T @ b
        b = rnd(rows * world, 384)
        h = ws.begin_gather(x)
        dw = ws.gemm(h.full, b, True, True, gather=h, bcast=True, dep="a")
        ws.release(h)
        ok &= close(dw, full.float().t() @ b.float(), 2e-2, f"wgrad_a it{it}")
        # ---- ... and on the B side, accumulating into fp32:  dW[M2, K] += a^T @ full
        a = rnd(rows * world, 256)
        acc = torch.ones(256, K, device=dev, dtype=torch.float32)
        h = ws.begin_gather(x)
        ws.gemm(a, h.full, True, True, out=acc, add=acc, gather=h, bcast=True, dep="b")
        ws.release(h)
        ok &= close(acc, 1.0 + a.float().t() @ full.float(), 2e-2, f"wgrad_b it{it}")
        # ---- stand-alone all-gather by peer loads
        ok &= bool(torch.equal(ws.all_gather(x), full))

        # ---- GEMM -> reduce-scatter, with post-reduction bias and residual
        xa = rnd(rows * world, K)
        wr = rnd(N, K, scale=0.05)
        bias = rnd(N)
        res = rnd(rows, N)
        part = (xa.float() @ wr.float().t()).to(torch.bfloat16).float()
        ref = torch.empty(rows, N, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(ref, part.contiguous(), group=grp)
        out = ws.gemm_reduce(xa, wr, False, bias=bias, residual=res)
        ok &= close(out, ref + bias.float() + res.float(), 2e-2, f"gemm_rs it{it}")
        # ---- GEMM -> all-reduce with per-rank (pre-reduction) bias and addend
        padd = rnd(rows * world, N)
        part2 = (xa.float() @ wr.float().t() + bias.float() + padd.float()).to(torch.bfloat16).float()
        dist.all_reduce(part2, group=grp)
        out2 = ws.gemm_reduce(xa, wr, False, all_reduce=True, partial_bias=bias, partial_add=padd)
        ok &= close(out2, part2, 2e-2, f"gemm_ar it{it}")
        # ---- dgrad form (MN-major B) -> reduce-scatter
        dy = rnd(rows * world, N)
        part3 = (dy.float() @ wr.float()).to(torch.bfloat16).float()
        ref3 = torch.empty(rows, K, device=dev, dtype=torch.float32)
        dist.reduce_scatter_tensor(ref3, part3.contiguous(), group=grp)
        h = ws.begin_gather(x)
        out3 = ws.gemm_reduce(dy, wr, True, gather=h)                 # the broadcast rides along as a prefetch
        ok &= close(out3, ref3, 2e-2, f"gemm_rs(b_mn) it{it}")
        dw3 = ws.gemm(a, h.full, True, True, gather=h, dep="b")       # ... for this GEMM, which only checks arrival
        ws.release(h)
        ok &= close(dw3, a.float().t() @ full.float(), 2e-2, f"prefetched wgrad it{it}")

    st = native.read_status()
    if st != 0:
        print(f"[rank {rank}] device status {st}", flush=True)
        ok = False

    # ---- layer level: fused vs NCCL formulation of column -> row parallel linears, forward and backward
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from common import make_args
    from gpt_neox_b200.parallel.layers import ColumnParallelLinear, RowParallelLinear
    from gpt_neox_b200.parallel.rng import model_parallel_cuda_manual_seed
    model_parallel_cuda_manual_seed(4321)
    for sp, fused_ag in ((True, "1"), (True, "0"), (False, "0")):
        os.environ["NEOX_FUSED_AG"] = fused_ag
        args = make_args(hidden_size=512, num_attention_heads=8, seq_length=128 * world,
                         max_position_embeddings=128 * world, precision="bfloat16", model_parallel_size=world,
                         sequence_parallel=sp, train_micro_batch_size_per_gpu=4, global_num_gpus=world,
                         distributed_backend="nccl")
        torch.manual_seed(7)
        col = ColumnParallelLinear(args, 512, 2048, gather_output=False, skip_bias_add=False)
        row = RowParallelLinear(args, 2048, 512, input_is_parallel=True, skip_bias_add=False)
        s, b = 128 * world, 4
        xs = rnd(s // world if sp else s, b, 512)
        if not sp:
            dist.broadcast(xs, 0)
        results = {}
        for mode in ("1", "0"):
            os.environ["NEOX_FUSED_TP_COMM"] = mode
            for p in list(col.parameters()) + list(row.parameters()):
                p.grad = None
            xin = xs.clone().requires_grad_(True)
            h, _ = col(xin, act=None)
            o, _ = row(h)
            (o.float() * 0.01).sum().backward()
            results[mode] = [o.detach(), xin.grad] + [p.grad for p in list(col.parameters()) + list(row.parameters())]
        os.environ["NEOX_FUSED_TP_COMM"] = "1"
        for i, (fa, fb) in enumerate(zip(results["1"], results["0"])):
            ok &= close(fa, fb, 3e-2, f"layer sp={sp} tensor{i}")
    st = native.read_status()
    if st != 0:
        print(f"[rank {rank}] device status {st} after layer test", flush=True)
        ok = False

    # ---- vocabulary-parallel cross entropy (single-pass statistics re-based on the global maximum) vs the dense loss
    from gpt_neox_b200.parallel.cross_entropy import vocab_parallel_cross_entropy
    V = 1024 * world
    full_logits = (torch.randn(96, V, device=dev, generator=torch.Generator(device=dev).manual_seed(77)) * 4).to(torch.bfloat16)
    tgt = torch.randint(0, V, (96,), device=dev, generator=torch.Generator(device=dev).manual_seed(78))
    shard_l = full_logits[:, rank * 1024:(rank + 1) * 1024].contiguous().requires_grad_(True)
    loss = vocab_parallel_cross_entropy(shard_l, tgt)
    loss.sum().backward()
    ref_l = full_logits.float().requires_grad_(True)
    ref_loss = torch.nn.functional.cross_entropy(ref_l, tgt, reduction="none")
    ref_loss.sum().backward()
    ok &= close(loss, ref_loss, 2e-3, "vocab-parallel CE loss")
    ok &= close(shard_l.grad, ref_l.grad[:, rank * 1024:(rank + 1) * 1024], 2e-2, "vocab-parallel CE grad")

    # ---- bounded wait: nobody publishes this epoch, the gather must give up, report, and leave the context usable
    if os.environ.get("NEOX_TEST_TIMEOUT_PATH", "1") == "1":
        ws.gather(ws.ag_epoch + 1000, rows, K, last_reader=False)
        st = native.read_status()
        ok &= (520 <= st < 528)
        z = torch.ones(4, device=dev).sum().item()
        ok &= (z == 4.0)

    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0 and flag.item() == 1:
        print("FUSED_COMM_OK", flush=True)
    dist.barrier()
    fused_comm.reset()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
