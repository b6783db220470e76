"""Micro-benchmark: ZeRO-1 bucket traffic through the peer-memory kernels against NCCL.

Run one process per GPU::

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m gpt_neox_b200.parallel.bench_zero_peer --mib 256 1024

For every bucket size it times, call by call interleaved (CUDA events, median, max over ranks; the buffers are larger
than L2):

* reduce-scatter of an fp32 gradient bucket: ``dist.reduce_scatter_tensor`` against "raise READY, wait for the peers'
  READY, ``zero_reduce_scatter_kernel``" (the shard owner reads its shard from every rank and adds in rank order);
* all-gather of the updated 16-bit parameters: ``dist.all_gather_into_tensor`` against ``zero_param_push_kernel`` +
  the consumer's flag wait;

checks that both forms give the same numbers, and reports the achieved NVLink rate: every rank receives
``(world - 1) / world`` of the bucket in either direction of the exchange.
"""
import argparse
import ctypes
import json
import os

import torch
import torch.distributed as dist

from ..ops import native
from . import symm_mem as S

READY, DONE, GATHERED = 0, 8, 16


def median_interleaved(fns, iters):
    for fn in fns:
        for _ in range(3):
            fn()
    torch.cuda.synchronize()
    dist.barrier()
    ev = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
          for _ in fns]
    for i in range(iters):
        for k, fn in enumerate(fns):
            dist.barrier()                      # both forms start from aligned ranks
            s, e = ev[k][i]
            s.record()
            fn()
            e.record()
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
    ap.add_argument("--mib", type=int, nargs="+", default=[256, 1024], help="fp32 gradient bucket sizes in MiB")
    ap.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    L = native.lib()
    st = lambda: ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    rows = []
    for mib in a.mib:
        n = mib * (1 << 20) // 4
        n -= n % (8 * world)
        shard = n // world
        lo = shard * rank
        sym_g = S.SymmBuffer(n * 4)
        sym_p = S.SymmBuffer(n * 2)
        pad = S.SignalPad()
        ctr = torch.zeros(4, dtype=torch.int32, device="cuda")
        grad = sym_g.tensor((n,), torch.float32)
        param = sym_p.tensor((n,), torch.bfloat16)
        gen = torch.Generator(device="cuda").manual_seed(17 + rank)
        src = torch.randn(n, device="cuda", generator=gen)
        nccl_out = torch.empty(shard, device="cuda")
        epoch = [0]

        def rs_nccl():
            dist.reduce_scatter_tensor(nccl_out, src)

        def rs_peer():
            epoch[0] += 1
            e = ctypes.c_uint(epoch[0])
            native.check(L.neox_symm_release(None, 0, pad.c_ptrs, world, rank, READY, e, st()), "release")
            native.check(L.neox_wait_flags_long(pad.word(READY), e, world, rank, 5, st()), "wait")
            native.check(L.neox_zero_reduce_scatter(sym_g.c_ptrs, ctypes.c_ulonglong(lo), ctypes.c_ulonglong(shard),
                                                    ctypes.c_float(1.0), pad.word(READY), e, pad.c_ptrs, world, rank,
                                                    DONE, ctypes.c_void_p(ctr.data_ptr()), st()), "reduce_scatter")
            # what the optimizer does before it rewrites the buffer: everybody has finished reading it
            native.check(L.neox_wait_flags_long(pad.word(DONE), e, world, rank, 5, st()), "wait done")

        grad.copy_(src)
        torch.cuda.synchronize()
        dist.barrier()
        # correctness of one round, then timing (later rounds re-reduce the same buffer: the own shard then holds
        # running sums, which changes the values but not the traffic)
        rs_nccl()
        epoch[0] += 1
        e = ctypes.c_uint(epoch[0])
        L.neox_symm_release(None, 0, pad.c_ptrs, world, rank, READY, e, st())
        L.neox_wait_flags_long(pad.word(READY), e, world, rank, 5, st())
        L.neox_zero_reduce_scatter(sym_g.c_ptrs, ctypes.c_ulonglong(lo), ctypes.c_ulonglong(shard), ctypes.c_float(1.0),
                                   pad.word(READY), e, pad.c_ptrs, world, rank, DONE, ctypes.c_void_p(ctr.data_ptr()), st())
        L.neox_wait_flags_long(pad.word(DONE), e, world, rank, 5, st())
        torch.cuda.synchronize()
        err = (grad[lo:lo + shard] - nccl_out).abs().max().item()
        scale = nccl_out.abs().max().item()
        assert err <= 1e-5 * max(scale, 1.0) * world, (err, scale)
        t_nccl, t_peer = median_interleaved([rs_nccl, rs_peer], a.iters)

        # ---- all-gather of the 16-bit parameters
        pshard = torch.randn(shard, device="cuda", generator=gen).to(torch.bfloat16)
        full = torch.empty(n, dtype=torch.bfloat16, device="cuda")
        gepoch = [0]

        def ag_nccl():
            dist.all_gather_into_tensor(full, pshard)

        def ag_peer():
            gepoch[0] += 1
            e = ctypes.c_uint(gepoch[0])
            native.check(L.neox_zero_param_push(sym_p.c_ptrs, ctypes.c_ulonglong(lo * 2), ctypes.c_ulonglong(shard * 2),
                                                pad.c_ptrs, world, rank, GATHERED, e,
                                                ctypes.c_void_p(ctr.data_ptr() + 4), st()), "push")
            native.check(L.neox_wait_flags_long(pad.word(GATHERED), e, world, rank, 5, st()), "wait")

        param[lo:lo + shard].copy_(pshard)
        torch.cuda.synchronize()
        dist.barrier()
        ag_nccl()
        ag_peer()
        torch.cuda.synchronize()
        assert torch.equal(param, full)
        g_nccl, g_peer = median_interleaved([ag_nccl, ag_peer], a.iters)
        status = native.read_status()
        recv_rs = (world - 1) / world * n * 4
        recv_ag = (world - 1) / world * n * 2
        rows.append({"bucket_mib": mib, "world": world, "status": status,
                     "reduce_scatter_ms": {"nccl": round(t_nccl, 3), "peer": round(t_peer, 3)},
                     "reduce_scatter_gbs_in": {"nccl": round(recv_rs / t_nccl / 1e6, 1), "peer": round(recv_rs / t_peer / 1e6, 1)},
                     "all_gather_ms": {"nccl": round(g_nccl, 3), "peer": round(g_peer, 3)},
                     "all_gather_gbs_in": {"nccl": round(recv_ag / g_nccl / 1e6, 1), "peer": round(recv_ag / g_peer / 1e6, 1)}})
        torch.cuda.synchronize()
        dist.barrier()
        for b in (sym_g, sym_p, pad):
            b.close()
    if rank == 0:
        for r in rows:
            print(json.dumps(r), flush=True)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
