"""Stand-alone timing of the flash-attention kernels (forward, backward) on one GPU.

    python -m gpt_neox_b200.ops.bench_attention --seq 2048 --batch 4 --heads 64 --dim 96 [--iters 10]

Prints CUDA-event times and achieved TFLOP/s (causal FLOPs: forward 4*s^2*d*b*h/2, backward 2.5x that) for this
package's kernels and, for reference, torch SDPA on the same inputs.  Also the entry point used for ncu captures.
"""
import argparse
import json

import torch

from . import attention as A


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=64)
    ap.add_argument("--dim", type=int, default=96)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-sdpa", action="store_true")
    a = ap.parse_args()
    dev = torch.device("cuda")
    s, b, h, d = a.seq, a.batch, a.heads, a.dim
    mixed = torch.randn(s, b, h, 3 * d, device=dev, dtype=torch.bfloat16, requires_grad=True)
    q, k, v = mixed[..., :d], mixed[..., d:2 * d], mixed[..., 2 * d:]
    flops = 4.0 * s * s * d * b * h / 2

    def timeit(fn, n):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / n

    out = A.flash_attention(q, k, v)
    g = torch.randn_like(out)
    t_f = timeit(lambda: A.flash_attention(q, k, v), a.iters)

    def fb():
        mixed.grad = None
        o = A.flash_attention(q, k, v)
        o.backward(g)
    t_fb = timeit(fb, a.iters)
    res = {"shape": {"seq": s, "batch": b, "heads": h, "dim": d}, "fwd_ms": round(t_f, 4),
           "fwd_tflops": round(flops / t_f / 1e9, 1), "bwd_ms": round(t_fb - t_f, 4),
           "bwd_tflops": round(2.5 * flops / (t_fb - t_f) / 1e9, 1)}
    if not a.no_sdpa:
        qs, ks, vs = (t.detach().permute(1, 2, 0, 3).contiguous().requires_grad_(True) for t in (q, k, v))
        F = torch.nn.functional
        t_sf = timeit(lambda: F.scaled_dot_product_attention(qs, ks, vs, is_causal=True), a.iters)
        gs = g.permute(1, 2, 0, 3).contiguous()

        def sfb():
            o = F.scaled_dot_product_attention(qs, ks, vs, is_causal=True)
            o.backward(gs)
        t_sfb = timeit(sfb, a.iters)
        res.update({"sdpa_fwd_ms": round(t_sf, 4), "sdpa_fwd_tflops": round(flops / t_sf / 1e9, 1),
                    "sdpa_bwd_ms": round(t_sfb - t_sf, 4),
                    "sdpa_bwd_tflops": round(2.5 * flops / (t_sfb - t_sf) / 1e9, 1)})
    print(json.dumps(res))


if __name__ == "__main__":
    main()
