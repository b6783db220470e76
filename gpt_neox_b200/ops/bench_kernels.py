"""Roofline check of the single-GPU kernels: achieved bandwidth / throughput against the measured peaks.

    python -m gpt_neox_b200.ops.bench_kernels [--only gemm_fwd,layernorm_fwd,...] [--tokens 8192] [--hidden 6144]

Every entry is timed with CUDA events after warm-up with a 256 MiB buffer rewritten between iterations (L2 flush), and
reported as ``algorithmic bytes (or FLOPs) / time`` and as a fraction of the measured copy bandwidth / cuBLAS bf16
throughput (``MEASURED_PEAKS.json`` at the repository root when present, else 6650 GB/s and 1590 TFLOP/s).
The same entry points are what the ncu summaries under ``profiles/`` were captured from (``--only`` selects one).
"""
import argparse
import json
import os

import torch

from . import functional as OF
from . import gemm as G


def peaks():
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    try:
        p = json.load(open(os.path.join(root, "MEASURED_PEAKS.json")))
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except Exception:
        return 6650.0, 1590.0, "fallback"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--only", default="")
    ap.add_argument("--tokens", type=int, default=8192)
    ap.add_argument("--hidden", type=int, default=6144)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--ab-gemm", action="store_true",
                    help="only the five GEMM shapes, three ways taking turns call by call: one-CTA kernel, CTA-pair "
                         "kernel, cuBLAS through torch (F.linear / matmul, plus the element-wise kernels the fused "
                         "epilogues replace)")
    ap.add_argument("--moe", action="store_true",
                    help="only the mixture-of-experts kernels: router, dispatch / combine, and the grouped expert "
                         "GEMMs (forward, dgrad, wgrad) against the per-expert loop over the plain GEMM; "
                         "--tokens rows x top-2 of --experts experts, hidden --hidden, expert hidden --ffn")
    ap.add_argument("--small-kernels", action="store_true",
                    help="only the remaining element-wise / recurrent / optimizer kernels, each against its eager "
                         "torch statement: bias-dropout-residual, RoPE, embedding fwd/bwd, bias-gradient column sum, "
                         "wkv6, selective scan, top-k/top-p filter, Lion, block-wise 8-bit Adam, squared norm")
    ap.add_argument("--experts", type=int, default=8)
    ap.add_argument("--ffn", type=int, default=0, help="expert hidden size (default 4 x hidden)")
    a = ap.parse_args()
    only = set(x for x in a.only.split(",") if x)
    dev = torch.device("cuda")
    T, h = a.tokens, a.hidden
    hbm, tf, kind = peaks()
    flush = torch.zeros(64 << 20, device=dev)
    bf = lambda *s: (torch.randn(*s, device=dev) * 0.05).to(torch.bfloat16)
    out = []

    def run(name, fn, nbytes=0.0, flops=0.0):
        if only and name not in only:
            return
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.iters):
            flush.add_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ms = sorted(ts)[len(ts) // 2]
        rec = {"kernel": name, "ms": round(ms, 4)}
        if nbytes:
            rec["gbs"] = round(nbytes / ms / 1e6, 1)
            rec[f"of_{kind}_hbm"] = round(nbytes / ms / 1e6 / hbm, 3)
        if flops:
            rec["tflops"] = round(flops / ms / 1e9, 1)
            rec[f"of_{kind}_bf16"] = round(flops / ms / 1e9 / tf, 3)
        out.append(rec)
        print(json.dumps(rec), flush=True)

    if a.ab_gemm:
        return ab_gemm(a, dev, bf, flush)
    if a.moe:
        return moe_kernels(a, dev, bf, flush)
    if a.small_kernels:
        return small_kernels(a, dev, bf, flush)
    x = bf(T, h)
    w_qkv, w_fc1, w_fc2 = bf(3 * h, h), bf(4 * h, h), bf(h, 4 * h)
    y4 = bf(T, 4 * h)
    g_h = bf(T, h)
    acc = torch.zeros(4 * h, h, device=dev, dtype=torch.float32)
    bias4 = bf(4 * h)
    run("gemm_fwd_qkv", lambda: G.gemm(x, w_qkv), flops=2.0 * T * h * 3 * h)
    run("gemm_fwd_fc1_bias_gelu", lambda: G.gemm(x, w_fc1, bias=bias4, act=G.ACT_GELU, want_preact=True),
        flops=2.0 * T * h * 4 * h)
    run("gemm_fwd_fc2", lambda: G.gemm(y4, w_fc2), flops=2.0 * T * h * 4 * h)
    run("gemm_dgrad_fc1", lambda: G.gemm(y4, w_fc1, b_mn=True), flops=2.0 * T * h * 4 * h)
    run("gemm_wgrad_fc1_fp32_accumulate", lambda: G.gemm(y4, x, a_mn=True, b_mn=True, out=acc, add=acc),
        flops=2.0 * T * h * 4 * h)

    # the same five GEMMs through the CTA-pair kernel (cta_group::2)
    def paired(fn):
        def run_it():
            old = G._PAIR
            G._PAIR = "1"
            try:
                return fn()
            finally:
                G._PAIR = old
        return run_it

    run("pair_gemm_fwd_qkv", paired(lambda: G.gemm(x, w_qkv)), flops=2.0 * T * h * 3 * h)
    run("pair_gemm_fwd_fc1_bias_gelu", paired(lambda: G.gemm(x, w_fc1, bias=bias4, act=G.ACT_GELU, want_preact=True)),
        flops=2.0 * T * h * 4 * h)
    run("pair_gemm_fwd_fc2", paired(lambda: G.gemm(y4, w_fc2)), flops=2.0 * T * h * 4 * h)
    run("pair_gemm_dgrad_fc1", paired(lambda: G.gemm(y4, w_fc1, b_mn=True)), flops=2.0 * T * h * 4 * h)
    run("pair_gemm_wgrad_fc1_fp32_accumulate", paired(lambda: G.gemm(y4, x, a_mn=True, b_mn=True, out=acc, add=acc)),
        flops=2.0 * T * h * 4 * h)

    # fp8 tensor cores (per-tensor scaling): the three GEMMs of fc1 and the casts that feed them
    from . import fp8 as F8
    if not only or any(n.startswith("fp8_") for n in only):
        xq, wq, yq = F8.cast(x), F8.cast(w_fc1), F8.cast(y4, e5m2=True)
        run("fp8_gemm_fwd_fc1", lambda: F8.gemm_fp8(xq, wq), flops=2.0 * T * h * 4 * h)
        run("fp8_gemm_dgrad_fc1", lambda: F8.gemm_fp8(yq, wq, b_mn=True), flops=2.0 * T * h * 4 * h)
        run("fp8_gemm_wgrad_fc1_fp32_accumulate", lambda: F8.gemm_fp8(yq, xq, a_mn=True, b_mn=True, out=acc, add=acc),
            flops=2.0 * T * h * 4 * h)
        run("fp8_cast_current_T_x_4h", lambda: F8.cast(y4, e5m2=True), nbytes=(2 + 2 + 1.0) * T * 4 * h)
        lin_x = x.clone().requires_grad_(True)
        lin_w = torch.nn.Parameter(w_fc1.clone())
        rec = F8.Fp8Recipe()

        def lin_fp8():
            F8.fp8_linear(lin_x, lin_w, None, rec).backward(y4)
            lin_x.grad = lin_w.grad = None

        def lin_bf16():
            from .linear import linear
            linear(lin_x, lin_w, None).backward(y4)
            lin_x.grad = lin_w.grad = None

        run("fp8_linear_fc1_fwd_bwd", lin_fp8, flops=6.0 * T * h * 4 * h)
        run("fp8_ref_bf16_linear_fc1_fwd_bwd", lin_bf16, flops=6.0 * T * h * 4 * h)

    # MXFP8 on the block-scaled tensor cores
    from . import mxfp8 as MX
    if not only or any(n.startswith("mx_") for n in only):
        xm, wm = MX.quantize_tiled(x, False), MX.quantize_tiled(w_fc1, False)
        ym, wm_r = MX.quantize_tiled(y4, False, True), MX.quantize_tiled(w_fc1, True)
        ym_r, xm_r = MX.quantize_tiled(y4, True, True), MX.quantize_tiled(x, True)
        run("mx_gemm_fwd_fc1", lambda: MX.gemm_mx(xm, wm), flops=2.0 * T * h * 4 * h)
        run("mx_gemm_dgrad_fc1", lambda: MX.gemm_mx(ym, wm_r), flops=2.0 * T * h * 4 * h)
        run("mx_gemm_wgrad_fc1_fp32_accumulate", lambda: MX.gemm_mx(ym_r, xm_r, out=acc, add=acc),
            flops=2.0 * T * h * 4 * h)
        run("mx_quant_T_x_4h_along_cols", lambda: MX.quantize_tiled(y4, False, True), nbytes=(2 + 1.03) * T * 4 * h)
        run("mx_quant_T_x_4h_along_rows", lambda: MX.quantize_tiled(y4, True, True), nbytes=(2 + 1.03) * T * 4 * h)
        run("mx_quant_T_x_4h_both_directions_one_pass", lambda: MX.quantize_dual(y4, True), nbytes=(2 + 2.06) * T * 4 * h)
        run("mx_quant_T_x_4h_one_pass_cols_only", lambda: MX.quantize_dual(y4, True, rows=False),
            nbytes=(2 + 1.03) * T * 4 * h)
        mlin_x = x.clone().requires_grad_(True)
        mlin_w = torch.nn.Parameter(w_fc1.clone())

        def lin_mx(hw):
            def f():
                MX.mx_linear(mlin_x, mlin_w, None, hardware=hw).backward(y4)
                mlin_x.grad = mlin_w.grad = None
            return f

        run("mx_linear_fc1_fwd_bwd_hardware", lin_mx(True), flops=6.0 * T * h * 4 * h)
        run("mx_linear_fc1_fwd_bwd_emulated", lin_mx(False), flops=6.0 * T * h * 4 * h)

    gamma, beta = bf(h), bf(h)
    run("layernorm_fwd", lambda: OF.layer_norm(x, gamma, beta, 1e-5), nbytes=2.0 * T * h * 2)
    xl = x.clone().requires_grad_(True)
    gl, bl = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    yl = OF.layer_norm(xl, gl, bl, 1e-5)
    run("layernorm_bwd", lambda: torch.autograd.grad(yl, (xl, gl, bl), g_h, retain_graph=True),
        nbytes=3.0 * T * h * 2)
    run("rmsnorm_fwd", lambda: OF.rms_norm(x, gamma, None, 1e-6), nbytes=2.0 * T * h * 2)
    run("bias_gelu_fwd", lambda: OF.bias_gelu(y4, bias4), nbytes=2.0 * T * 4 * h * 2)
    sw = bf(T, 8 * h // 3 // 64 * 64 * 2)
    run("swiglu_fwd", lambda: OF.gated_act(sw, "swiglu"), nbytes=1.5 * sw.numel() * 2)
    sc = bf(4, 16, 2048, 2048)
    run("causal_softmax_fwd", lambda: OF.scaled_upper_triang_masked_softmax(sc.view(-1, 2048, 2048), 1.0),
        nbytes=2.0 * sc.numel() * 2)
    scg = sc.view(-1, 2048, 2048).detach().requires_grad_(True)
    ysm = OF.scaled_upper_triang_masked_softmax(scg, 1.0)
    gsm = torch.randn_like(ysm)
    run("causal_softmax_bwd", lambda: torch.autograd.grad(ysm, scg, gsm, retain_graph=True), nbytes=3.0 * sc.numel() * 2)
    V = 50432
    logits = bf(T, V)
    tgt = torch.randint(0, V, (T,), device=dev)
    from ..parallel.cross_entropy import vocab_parallel_cross_entropy
    run("cross_entropy_fwd", lambda: vocab_parallel_cross_entropy(logits, tgt), nbytes=2.0 * T * V * 2)
    n = 400 * 1000 * 1000
    p32, m32, v32, g32 = (torch.zeros(n, device=dev) for _ in range(4))
    pb = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    import ctypes
    from . import native

    def adam():
        rc = native.lib().neox_adam_step(native.ptr(p32), native.ptr(m32), native.ptr(v32), native.ptr(g32),
                                         native.ptr(pb), 0, ctypes.c_longlong(n), ctypes.c_float(1e-4),
                                         ctypes.c_float(0.9), ctypes.c_float(0.95), ctypes.c_float(1e-8),
                                         ctypes.c_float(0.01), ctypes.c_float(0.1), ctypes.c_float(0.05),
                                         ctypes.c_float(1.0), 1, ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_adam_step")
    run("adam_step_bf16_writeback", adam, nbytes=n * (4 * 4 + 3 * 4 + 2.0))
    if not only:
        print(json.dumps({"peaks": {"hbm_gbs": hbm, "bf16_tflops": tf, "kind": kind}, "results": out}))


def ab_gemm(a, dev, bf, flush):
    """Interleaved A/B/C of the GEMM kernels against cuBLAS on identical shapes: the variants take turns call by
    call (L2 flushed before every call), so all of them see the same clocks and power state; medians are reported."""
    import torch.nn.functional as F
    T, h = a.tokens, a.hidden
    x, y4, g_h = bf(T, h), bf(T, 4 * h), bf(T, h)
    w_qkv, w_fc1, w_fc2, bias4 = bf(3 * h, h), bf(4 * h, h), bf(h, 4 * h), bf(4 * h)
    acc = torch.zeros(4 * h, h, device=dev, dtype=torch.float32)

    def with_pair(flag, fn):
        def f():
            old, G._PAIR = G._PAIR, flag
            try:
                return fn()
            finally:
                G._PAIR = old
        return f

    def cublas_wgrad():
        acc.add_(y4.t() @ x)

    shapes = [
        ("fwd_qkv", 2.0 * T * h * 3 * h, lambda: G.gemm(x, w_qkv), lambda: F.linear(x, w_qkv)),
        ("fwd_fc1_bias_gelu", 2.0 * T * h * 4 * h, lambda: G.gemm(x, w_fc1, bias=bias4, act=G.ACT_GELU, want_preact=True),
         lambda: F.gelu(F.linear(x, w_fc1, bias4), approximate="tanh")),
        ("fwd_fc2", 2.0 * T * h * 4 * h, lambda: G.gemm(y4, w_fc2), lambda: F.linear(y4, w_fc2)),
        ("dgrad_fc1", 2.0 * T * h * 4 * h, lambda: G.gemm(y4, w_fc1, b_mn=True), lambda: y4 @ w_fc1),
        ("wgrad_fc1_fp32_accumulate", 2.0 * T * h * 4 * h,
         lambda: G.gemm(y4, x, a_mn=True, b_mn=True, out=acc, add=acc), cublas_wgrad),
    ]
    results = []
    for name, flops, ours, lib in shapes:
        fns = {"one_cta": with_pair("0", ours), "cta_pair": with_pair("1", ours), "cublas": lib}
        for f in fns.values():
            for _ in range(3):
                f()
        torch.cuda.synchronize()
        ts = {k: [] for k in fns}
        for _ in range(a.iters):
            for k, f in fns.items():
                flush.add_(1.0)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                f()
                e1.record()
                torch.cuda.synchronize()
                ts[k].append(e0.elapsed_time(e1))
        med = {k: sorted(v)[len(v) // 2] for k, v in ts.items()}
        rec = {"gemm": name, **{f"{k}_ms": round(v, 4) for k, v in med.items()},
               **{f"{k}_tflops": round(flops / v / 1e9, 1) for k, v in med.items()},
               "pair_over_cublas": round(med["cublas"] / med["cta_pair"], 3)}
        results.append(rec)
        print(json.dumps(rec), flush=True)
    return results


def _ab(name, fns, iters, flush, nbytes=0.0, extra=None):
    """Median time of every callable in ``fns`` (name -> fn), taking turns call by call, L2 flushed before each.
    A case whose set-up or first call raises is reported and skipped, so the remaining cases still run."""
    try:
        return _ab_run(name, fns, iters, flush, nbytes, extra)
    except Exception as exc:      # noqa: BLE001 -- a benchmark driver: report and go on
        rec = {"kernel": name, "error": f"{type(exc).__name__}: {exc}"[:300]}
        print(json.dumps(rec), flush=True)
        return rec


def _ab_run(name, fns, iters, flush, nbytes, extra):
    hbm, _, kind = peaks()
    for f in fns.values():
        for _ in range(3):
            f()
    torch.cuda.synchronize()
    ts = {k: [] for k in fns}
    for _ in range(iters):
        for k, f in fns.items():
            flush.add_(1.0)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            f()
            e1.record()
            torch.cuda.synchronize()
            ts[k].append(e0.elapsed_time(e1))
    med = {k: sorted(v)[len(v) // 2] for k, v in ts.items()}
    keys = list(med)
    rec = {"kernel": name, **{f"{k}_ms": round(v, 4) for k, v in med.items()}}
    if len(keys) == 2:
        rec["speedup"] = round(med[keys[0]] / med[keys[1]], 2)
    if nbytes:
        rec["gbs"] = round(nbytes / med[keys[-1]] / 1e6, 1)
        rec[f"frac_of_{kind}_copy_bw"] = round(nbytes / med[keys[-1]] / 1e6 / hbm, 3)
    rec.update(extra or {})
    print(json.dumps(rec), flush=True)
    return rec


def small_kernels(a, dev, bf, flush):
    """The kernels that the other modes do not time, each against the eager torch statement of the same operation."""
    import torch.nn.functional as F
    from ..optim.adam8bit import Adam8bit
    from ..optim.lion import Lion
    from ..text_generation import filter_logits
    from . import embedding as E
    from . import selective_scan as SS
    from . import wkv6 as W
    T, h, it = a.tokens, a.hidden, a.iters
    out = []
    x, res, bias = bf(T, h), bf(T, h), bf(h)
    out.append(_ab("bias_dropout_residual_fwd",
                   {"torch": lambda: res + F.dropout(x + bias, 0.1, True),
                    "kernel": lambda: OF.bias_dropout_add(x, bias, res, 0.1, True)}, it, flush, 3.0 * T * h * 2))
    q = bf(2048, 4, 64, 96)
    t = torch.arange(2048, device=dev).float()
    inv = 1.0 / (10000 ** (torch.arange(0, 24, 2, device=dev).float() / 24))
    emb = torch.cat([torch.outer(t, inv)] * 2, -1)
    cos, sin = emb.cos()[:, None, None, :], emb.sin()[:, None, None, :]
    out.append(_ab("rope_partial_24_of_96", {"torch": lambda: OF.rope_ref(q, cos, sin), "kernel": lambda: OF.rope(q, cos, sin)},
                   it, flush, 2.0 * q.numel() * 2))
    q2 = bf(2048, 4, 32, 128)
    inv2 = 1.0 / (10000 ** (torch.arange(0, 128, 2, device=dev).float() / 128))
    emb2 = torch.cat([torch.outer(t, inv2)] * 2, -1)
    cos2, sin2 = emb2.cos()[:, None, None, :], emb2.sin()[:, None, None, :]
    out.append(_ab("rope_full_128", {"torch": lambda: OF.rope_ref(q2, cos2, sin2), "kernel": lambda: OF.rope(q2, cos2, sin2)},
                   it, flush, 2.0 * q2.numel() * 2))
    V = 50432
    table = torch.nn.Parameter(bf(V, h))
    ids = torch.randint(0, V, (4, 2048), device=dev)
    out.append(_ab("embedding_fwd", {"torch": lambda: F.embedding(ids, table), "kernel": lambda: E.embedding(ids, table)},
                   it, flush, 2.0 * ids.numel() * h * 2))
    ge = bf(4, 2048, h)

    def emb_bwd(fn):
        def f():
            table.grad = None
            fn(ids, table).backward(ge)
        return f
    out.append(_ab("embedding_fwd_bwd", {"torch": emb_bwd(F.embedding), "kernel": emb_bwd(E.embedding)}, it, flush))
    g4 = bf(T, 4 * h)
    out.append(_ab("bias_grad_column_sum", {"torch": lambda: g4.sum(0), "kernel": lambda: OF.bias_grad(g4)}, it, flush,
                   T * 4 * h * 2.0))
    B_, T_, H_, N_ = 4, 1024, 32, 64
    r, k, v, w = (bf(B_, T_, H_ * N_) for _ in range(4))
    u = bf(H_, N_)
    out.append(_ab("wkv6_fwd", {"kernel": lambda: W.wkv6(r, k, v, w, u)}, it, flush, 5.0 * r.numel() * 2,
                   {"shape": [B_, T_, H_, N_]}))
    b_, l_, d_, n_ = 4, 2048, 4096, 16
    us, dts, zs = bf(b_, l_, d_), bf(b_, l_, d_), bf(b_, l_, d_)
    A = -torch.rand(d_, n_, device=dev) - 0.5
    Bm, Cm = bf(b_, l_, n_), bf(b_, l_, n_)
    D, dtb = torch.ones(d_, device=dev), torch.zeros(d_, device=dev)
    out.append(_ab("selective_scan_fwd", {"kernel": lambda: SS.selective_scan(us, dts, A, Bm, Cm, D, zs, dtb)}, it, flush,
                   4.0 * us.numel() * 2, {"shape": [b_, l_, d_, n_]}))
    lg = torch.randn(64, V, device=dev)

    def eager_filter():
        kth = torch.topk(lg, 50)[0][..., -1, None]
        x2 = lg.masked_fill(lg < kth, -float("inf"))
        sl, si = torch.sort(x2, descending=True, dim=-1)
        rm = torch.cumsum(F.softmax(sl, dim=-1), dim=-1) > 0.9
        rm[..., 1:] = rm[..., :-1].clone()
        rm[..., 0] = False
        return x2.masked_fill(torch.zeros_like(rm).scatter(-1, si, rm), -float("inf"))
    out.append(_ab("top_k_50_top_p_0.9_filter", {"torch": eager_filter, "kernel": lambda: filter_logits(lg, 50, 0.9)},
                   it, flush))
    n = 100 * 1000 * 1000
    p1, p2 = torch.nn.Parameter(torch.zeros(n, device=dev)), torch.nn.Parameter(torch.zeros(n, device=dev))
    p1.grad, p2.grad = torch.randn(n, device=dev), torch.randn(n, device=dev)
    lion, a8 = Lion([p1], lr=1e-4), Adam8bit([p2], lr=1e-4)
    out.append(_ab("lion_step_100M", {"kernel": lion.step}, it, flush, n * 4 * 5.0))
    out.append(_ab("adam8bit_step_100M", {"kernel": a8.step}, it, flush, n * (4 * 3 + 2 * 2.0)))
    tot = torch.zeros((), device=dev)
    import ctypes
    from . import native

    def sumsq():
        rc = native.lib().neox_sumsq_f32(native.ptr(p1.grad), ctypes.c_longlong(n), native.ptr(tot),
                                         ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_sumsq_f32")
    out.append(_ab("squared_norm_100M", {"torch": lambda: torch.linalg.vector_norm(p1.grad) ** 2, "kernel": sumsq}, it,
                   flush, n * 4.0))
    print(json.dumps({"status_word": native.read_status()}), flush=True)
    return out


def moe_kernels(a, dev, bf, flush):
    """Router, dispatch / combine and the grouped expert GEMMs against the per-expert loop, taking turns call by
    call (L2 flushed before every call); medians.  Assignments are drawn from a softmax over random logits, so the
    experts are unevenly loaded the way a real router loads them."""
    from . import moe_ops as MO
    T, h, E, k = a.tokens, a.hidden, a.experts, 2
    ffn = a.ffn or 4 * h
    hbm, tf, kind = peaks()
    x = bf(T, h)
    logits = (torch.randn(T, E, device=dev) * 1.5).to(torch.bfloat16)
    w1, w2 = bf(E, ffn, h), bf(E, h, ffn)
    probs, gate, idx, counts = MO.router(logits, k)
    row_of, kept = MO.plan_rows(idx, counts)
    rows = MO.padded_rows(T * k, E)
    xs = MO.dispatch(x, row_of, rows)
    g_out = torch.zeros(rows, ffn, device=dev, dtype=torch.bfloat16)
    g_out[row_of.reshape(-1)] = bf(T * k, ffn)
    segs = MO._segments(kept)
    acc = torch.zeros(E, ffn, h, device=dev, dtype=torch.float32)
    pre = torch.empty(rows, ffn, device=dev, dtype=torch.bfloat16)
    out_f, out_d = torch.empty(rows, ffn, device=dev, dtype=torch.bfloat16), torch.empty(rows, h, device=dev, dtype=torch.bfloat16)

    def loop_fwd():
        for e, (r, n) in enumerate(segs):
            if n:
                G.gemm(xs[r:r + n], w1[e], act=G.ACT_GELU, want_preact=True)

    def loop_dgrad():
        for e, (r, n) in enumerate(segs):
            if n:
                G.gemm(g_out[r:r + n], w1[e], b_mn=True)

    def loop_wgrad():
        for e, (r, n) in enumerate(segs):
            if n:
                G.gemm(g_out[r:r + n], xs[r:r + n], a_mn=True, b_mn=True, out=acc[e], add=acc[e])

    def grouped_fwd():
        MO._grouped_call(xs, w1, out_f, rows, ffn, h, h, h, ffn, False, kept, E, 1, preact=pre, act=G.ACT_GELU)

    def grouped_dgrad():
        MO._grouped_call(g_out, w1, out_d, rows, h, ffn, ffn, h, h, True, kept, E, 1)

    def grouped_wgrad():
        MO._grouped_call(g_out, xs, acc.view(E * ffn, h), ffn, h, rows, ffn, h, h, True, kept, E, 2,
                         add=acc.view(E * ffn, h))

    flops = 2.0 * T * k * h * ffn
    cases = [
        ("expert_fc1_fwd_gelu", flops, 0.0, {"per_expert_loop": loop_fwd, "grouped": grouped_fwd}),
        ("expert_fc1_dgrad", flops, 0.0, {"per_expert_loop": loop_dgrad, "grouped": grouped_dgrad}),
        ("expert_fc1_wgrad_fp32_accumulate", flops, 0.0, {"per_expert_loop": loop_wgrad, "grouped": grouped_wgrad}),
        ("router_softmax_top2", 0.0, T * E * (2 + 4) + T * k * 12.0,
         {"torch": lambda: MO.router_ref(logits, k), "kernel": lambda: MO.router(logits, k)}),
        ("dispatch_rows", 0.0, T * h * 2.0 + T * k * h * 2.0 + rows * h * 2.0,
         {"torch": lambda: MO.dispatch_ref(x, row_of, rows), "kernel": lambda: MO.dispatch(x, row_of, rows)}),
        ("combine_rows", 0.0, T * k * h * 2.0 + T * h * 2.0,
         {"torch": lambda: MO.combine_ref(out_d, row_of, gate), "kernel": lambda: MO.combine(out_d, row_of, gate)}),
    ]
    results = []
    for name, fl, nbytes, fns in cases:
        for f in fns.values():
            for _ in range(3):
                f()
        torch.cuda.synchronize()
        ts = {key: [] for key in fns}
        for _ in range(a.iters):
            for key, f in fns.items():
                flush.add_(1.0)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                f()
                e1.record()
                torch.cuda.synchronize()
                ts[key].append(e0.elapsed_time(e1))
        med = {key: sorted(v)[len(v) // 2] for key, v in ts.items()}
        rec = {"kernel": name, "tokens": T, "experts": E, "hidden": h, "ffn": ffn,
               **{f"{key}_ms": round(v, 4) for key, v in med.items()}}
        keys = list(med)
        rec["speedup"] = round(med[keys[0]] / med[keys[1]], 3)
        if fl:
            rec["tflops"] = round(fl / med[keys[1]] / 1e9, 1)
            rec[f"frac_of_{kind}_bf16_peak"] = round(fl / med[keys[1]] / 1e9 / tf, 3)
        if nbytes:
            rec["gbs"] = round(nbytes / med[keys[1]] / 1e6, 1)
            rec[f"frac_of_{kind}_copy_bw"] = round(nbytes / med[keys[1]] / 1e6 / hbm, 3)
        results.append(rec)
        print(json.dumps(rec), flush=True)
    from . import native
    print(json.dumps({"status_word": native.read_status(), "counts": kept.tolist()}), flush=True)
    return results


if __name__ == "__main__":
    main()
