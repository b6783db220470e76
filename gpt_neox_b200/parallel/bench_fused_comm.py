"""Micro-benchmark: fused GEMM+collective kernels against "NCCL collective, then GEMM" on transformer-layer shapes.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m gpt_neox_b200.parallel.bench_fused_comm --hidden 6144 --tokens 8192

For each of the four tensor-parallel GEMMs of a layer it reports, per launch (CUDA events, L2 flushed between
iterations, max over ranks): the GEMM alone, NCCL + GEMM back to back, the fused kernel(s), and the roofline target
``max(FLOPs / gemm_peak, NVLink bytes / link_bw)``.
"""
import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import gemm as G
from . import fused_comm, mpu


_skip = False


def timed(fn, iters, flush):
    if _skip:
        return float("nan")
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for i in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    for s, e in ev:
        flush.add_(1.0)
        s.record()
        fn()
        e.record()
    torch.cuda.synchronize()
    ts = sorted(s.elapsed_time(e) for s, e in ev)
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.item()


def timed_interleaved(fns, iters, flush):
    """Median time of every callable in ``fns``, the callables taking turns call by call: all of them see the same
    clocks and power state (back-to-back loops favour whichever runs first, while the GPU is still cool)."""
    if _skip:
        return [float("nan")] * len(fns)
    for fn in fns:
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
          for _ in fns]
    for i in range(iters):
        for k, fn in enumerate(fns):
            flush.add_(1.0)
            ev[k][i][0].record()
            fn()
            ev[k][i][1].record()
    torch.cuda.synchronize()
    out = []
    for k in range(len(fns)):
        ts = sorted(s.elapsed_time(e) for s, e in ev[k])
        t = torch.tensor([ts[len(ts) // 2]], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out.append(t.item())
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--hidden", type=int, default=6144)
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--only", type=str, default="", help="comma-separated op names to run (default: all)")
    ap.add_argument("--gemm-tflops", type=float, default=1406.8)
    ap.add_argument("--link-gbs", type=float, default=770.0)
    a = ap.parse_args()
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group("nccl")
    world, rank = dist.get_world_size(), dist.get_rank()
    mpu.initialize_model_parallel(world)
    grp = mpu.get_model_parallel_group()
    ws = fused_comm.workspace()
    dev = torch.device("cuda", torch.cuda.current_device())
    h, T = a.hidden, a.tokens
    rows = T // world
    flush = torch.zeros(64 << 20, device=dev)        # 256 MiB > L2
    rnd = lambda *s: (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)
    results = []

    only = set(x for x in a.only.split(",") if x)
    want = lambda name: not only or name in only

    def select(name):
        global _skip
        _skip = not want(name)

    def report(name, flops, link_bytes, t_gemm, t_nccl, t_fused):
        if not want(name):
            return
        target = max(flops / (a.gemm_tflops * 1e12), link_bytes / (a.link_gbs * 1e9)) * 1e3
        results.append({"op": name, "gemm_only_ms": round(t_gemm, 4), "nccl_then_gemm_ms": round(t_nccl, 4),
                        "fused_ms": round(t_fused, 4), "roofline_ms": round(target, 4),
                        "fused_of_roofline": round(target / t_fused, 3), "speedup_vs_nccl": round(t_nccl / t_fused, 3)})

    # ---- all-gather -> GEMM (column-parallel forward): qkv and fc1
    for name, n_out in (("ag_gemm_qkv", 3 * h // world), ("ag_gemm_fc1", 4 * h // world)):
        select(name)
        x, w = rnd(rows, h), rnd(n_out, h)
        full = torch.empty(T, h, device=dev, dtype=torch.bfloat16)

        def nccl():
            dist.all_gather_into_tensor(full, x, group=grp)
            return G.gemm(full, w)

        def fused():
            hd = ws.begin_gather(x)
            y = ws.gemm(hd.full, w, gather=hd, bcast=True, dep="a")
            ws.release(hd)
            return y

        t_g, t_n, t_f = timed_interleaved([lambda: G.gemm(full, w), nccl, fused], a.iters, flush)
        report(name, 2.0 * T * h * n_out, (world - 1) * rows * h * 2, t_g, t_n, t_f)

    # ---- GEMM -> reduce-scatter (row-parallel forward): attention dense and fc2
    for name, k_in in (("gemm_rs_dense", h // world), ("gemm_rs_fc2", 4 * h // world)):
        select(name)
        x, w = rnd(T, k_in), rnd(h, k_in)
        out = torch.empty(rows, h, device=dev, dtype=torch.bfloat16)

        def nccl():
            y = G.gemm(x, w)
            dist.reduce_scatter_tensor(out, y, group=grp)
            return out

        t_g, t_n, t_f = timed_interleaved([lambda: G.gemm(x, w), nccl, lambda: ws.gemm_reduce(x, w, False)], a.iters,
                                          flush)
        report(name, 2.0 * T * h * k_in, (world - 1) * rows * h * 2, t_g, t_n, t_f)

    # ---- GEMM -> all-reduce (row-parallel forward without sequence parallelism)
    select("gemm_ar_fc2")
    x, w = rnd(T, 4 * h // world), rnd(h, 4 * h // world)

    def nccl_ar():
        y = G.gemm(x, w)
        dist.all_reduce(y, group=grp)
        return y

    t_g, t_n, t_f = timed_interleaved([lambda: G.gemm(x, w), nccl_ar,
                                       lambda: ws.gemm_reduce(x, w, False, all_reduce=True)], a.iters, flush)
    report("gemm_ar_fc2", 2.0 * T * h * (4 * h // world), 2 * (world - 1) * rows * h * 2, t_g, t_n, t_f)

    # ---- weight gradient with the gathered operand (column-parallel backward)
    select("ag_wgrad_fc1")
    dy, xs = rnd(T, 4 * h // world), rnd(rows, h)
    full = torch.empty(T, h, device=dev, dtype=torch.bfloat16)
    acc = torch.zeros(4 * h // world, h, device=dev, dtype=torch.float32)

    def nccl_w():
        dist.all_gather_into_tensor(full, xs, group=grp)
        return G.gemm(dy, full, a_mn=True, b_mn=True, out=acc, add=acc)

    def fused_w():
        hd = ws.begin_gather(xs)
        ws.gemm(dy, hd.full, True, True, out=acc, add=acc, gather=hd, bcast=True, dep="b")
        ws.release(hd)

    t_g = timed(lambda: G.gemm(dy, full, a_mn=True, b_mn=True, out=acc, add=acc), a.iters, flush)
    report("ag_wgrad_fc1", 2.0 * T * h * (4 * h // world), (world - 1) * rows * h * 2, t_g, timed(nccl_w, a.iters, flush),
           timed(fused_w, a.iters, flush))

    # ---- diagnostics: the communication kernel without any job, and with the dependency only (data already there)
    select("wgrad_diag")

    def two():
        hd = ws.begin_gather(xs)
        ws.gemm(dy, hd.full, True, True, out=acc, add=acc, gather=hd, bcast=True, dep="b")
        ws.gemm(dy, hd.full, True, True, out=acc, add=acc, gather=hd, dep="b")
        ws.release(hd)

    report("wgrad_diag", 2.0 * T * h * (4 * h // world), 0.0,
           timed(lambda: ws.gemm(dy, full, True, True, out=acc, add=acc), a.iters, flush),
           timed(fused_w, a.iters, flush), timed(two, a.iters, flush))

    # ---- plain all-gather by peer loads (no GEMM): upper bound on what the in-kernel pull can reach
    select("all_gather_only")
    t_pull = timed(lambda: ws.all_gather(xs), a.iters, flush)
    t_ag = timed(lambda: dist.all_gather_into_tensor(full, xs, group=grp), a.iters, flush)
    report("all_gather_only", 0.0, (world - 1) * rows * h * 2, 0.0, t_ag, t_pull)

    # ---- whole column-parallel backward: dgrad -> reduce-scatter and wgrad with all-gathered x
    select("column_bwd_fc1")
    wc = rnd(4 * h // world, h)
    dxo = torch.empty(rows, h, device=dev, dtype=torch.bfloat16)

    def nccl_bwd():
        dist.all_gather_into_tensor(full, xs, group=grp)
        dx = G.gemm(dy, wc, b_mn=True)
        dist.reduce_scatter_tensor(dxo, dx, group=grp)
        return G.gemm(dy, full, a_mn=True, b_mn=True, out=acc, add=acc)

    def fused_bwd():
        hd = ws.begin_gather(xs)
        ws.gemm_reduce(dy, wc, True, gather=hd)
        ws.gemm(dy, hd.full, True, True, out=acc, add=acc, gather=hd, dep="b")
        ws.release(hd)

    def plain_bwd():
        G.gemm(dy, wc, b_mn=True)
        return G.gemm(dy, full, a_mn=True, b_mn=True, out=acc, add=acc)

    report("column_bwd_fc1", 4.0 * T * h * (4 * h // world), 2 * (world - 1) * rows * h * 2,
           timed(plain_bwd, a.iters, flush), timed(nccl_bwd, a.iters, flush), timed(fused_bwd, a.iters, flush))

    from ..ops import native
    st = native.read_status()
    if rank == 0:
        print(json.dumps({"world": world, "hidden": h, "tokens": T, "device_status": st, "gemm_peak_tflops": a.gemm_tflops,
                          "link_gbs": a.link_gbs, "results": results}, indent=1), flush=True)
    dist.barrier()
    fused_comm.reset()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
