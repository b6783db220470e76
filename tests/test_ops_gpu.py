"""Numerics of every CUDA kernel against the plain PyTorch fp32 statement of the same op."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpt_neox_b200.ops import functional as OF
from gpt_neox_b200.ops import gemm as G
from gpt_neox_b200.ops import native

DEV = "cuda"


def _close(a, b, atol, rtol=1e-2):
    a, b = a.float(), b.float()
    err = (a - b).abs()
    tol = atol + rtol * b.abs()
    assert bool((err <= tol).all()), f"max err {err.max().item():.4g} (tol {atol}, {rtol})"


@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(128, 256, 64, 0, 0), (256, 512, 256, 0, 1), (256, 512, 256, 1, 0),
                                             (384, 264, 136, 1, 1), (1000, 840, 328, 0, 0), (77, 96, 200, 0, 1)])
def test_gemm_layouts(M, N, K, a_mn, b_mn):
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    out = G.gemm(a, b, a_mn, b_mn)
    ref = G.gemm_ref(a, b, a_mn, b_mn, out_dtype=torch.float32)
    assert native.read_status() == 0
    _close(out, ref, atol=0.02 * ref.abs().max().item(), rtol=1e-2)


def test_gemm_epilogues():
    torch.manual_seed(1)
    M, N, K = 512, 1024, 512
    a = torch.randn(M, K, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(N, K, device=DEV, dtype=torch.bfloat16) * 0.05
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    res = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out, pre = G.gemm(a, b, bias=bias, act=G.ACT_GELU, add=res, want_preact=True)
    ro, rp = G.gemm_ref(a, b, bias=bias, act=G.ACT_GELU, add=res, want_preact=True, out_dtype=torch.float32)
    _close(out, ro, atol=0.05)
    _close(pre, rp, atol=0.05)
    aux = torch.randn(M, N, device=DEV, dtype=torch.bfloat16)
    out = G.gemm(a, b, act=G.ACT_DGELU, aux=aux)
    _close(out, G.gemm_ref(a, b, act=G.ACT_DGELU, aux=aux, out_dtype=torch.float32), atol=0.05)
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    want = G.gemm_ref(a, b, add=acc, out_dtype=torch.float32)
    G.gemm(a, b, out=acc, add=acc)
    _close(acc, want, atol=0.02)
    assert native.read_status() == 0


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
@pytest.mark.parametrize("rows,cols", [(33, 64), (128, 2048), (17, 6144), (5, 16384)])
def test_layernorm(dtype, rows, cols):
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(dtype).requires_grad_()
    b = (0.1 * torch.randn(cols, device=DEV)).to(dtype).requires_grad_()
    y = OF.layer_norm(x, w, b, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr, br = (t.detach().float().requires_grad_() for t in (x, w, b))
    yr = torch.nn.functional.layer_norm(xr, (cols,), wr, br, 1e-5)
    yr.backward(g.float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    _close(y, yr, tol)
    _close(x.grad, xr.grad, tol)
    _close(w.grad, wr.grad, tol * math.sqrt(rows), rtol=2e-2)
    _close(b.grad, br.grad, tol * math.sqrt(rows), rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("rows,cols", [(33, 64), (64, 4096)])
def test_rmsnorm(dtype, rows, cols):
    torch.manual_seed(0)
    x = torch.randn(rows, cols, device=DEV, dtype=dtype, requires_grad=True)
    w = (1 + 0.1 * torch.randn(cols, device=DEV)).to(dtype).requires_grad_()
    y = OF.rms_norm(x, w, None, 1e-5)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = (t.detach().float().requires_grad_() for t in (x, w))
    yr = OF.rms_norm_ref(xr, wr, None, 1e-5)
    yr.backward(g.float())
    tol = 1e-4 if dtype == torch.float32 else 3e-2
    _close(y, yr, tol)
    _close(x.grad, xr.grad, tol)
    _close(w.grad, wr.grad, tol * math.sqrt(rows), rtol=2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_bias_gelu_and_gated(dtype):
    torch.manual_seed(0)
    x = torch.randn(37, 512, device=DEV, dtype=dtype, requires_grad=True)
    bias = torch.randn(512, device=DEV, dtype=dtype, requires_grad=True)
    y = OF.bias_gelu(x, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr, br = x.detach().float().requires_grad_(), bias.detach().float().requires_grad_()
    yr = torch.nn.functional.gelu(xr + br, approximate="tanh")
    yr.backward(g.float())
    tol = 2e-3 if dtype == torch.float32 else 3e-2
    _close(y, yr, tol)
    _close(x.grad, xr.grad, tol)
    for kind in ("geglu", "swiglu", "reglu", "bilinear", "glu"):
        x2 = torch.randn(19, 256, device=DEV, dtype=dtype, requires_grad=True)
        y2 = OF.gated_act(x2, kind)
        g2 = torch.randn_like(y2)
        y2.backward(g2)
        x2r = x2.detach().float().requires_grad_()
        y2r = OF.gated_act_ref(x2r, kind)
        y2r.backward(g2.float())
        _close(y2, y2r, tol)
        _close(x2.grad, x2r.grad, tol)


@pytest.mark.parametrize("sk", [17, 128, 1000, 2048, 5000])
def test_softmax(sk):
    torch.manual_seed(0)
    b, h, sq = 2, 3, 8
    x = torch.randn(b, h, sq, sk, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    mask = torch.rand(b, 1, sq, sk, device=DEV) < 0.3
    y = OF.scaled_masked_softmax(x, mask, 0.7)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = OF.scaled_masked_softmax_ref(xr, mask, 0.7)
    yr.backward(g.float())
    # the reference bar for this kernel is a mean absolute difference <= 1e-3
    assert (y.float() - yr).abs().mean().item() <= 1e-3
    _close(y, yr, 1e-2)
    _close(x.grad, xr.grad, 2e-2)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("s", [16, 129, 2048])
def test_causal_softmax(s, dtype):
    torch.manual_seed(0)
    x = torch.randn(4, s, s, device=DEV, dtype=dtype, requires_grad=True)
    y = OF.scaled_upper_triang_masked_softmax(x, 0.5)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = OF.scaled_causal_softmax_ref(xr, 0.5)
    yr.backward(g.float())
    assert (y.float() - yr).abs().mean().item() <= 1e-3
    assert bool((y.float().triu(1) == 0).all())
    _close(x.grad, xr.grad, 2e-2)


@pytest.mark.parametrize("d,rot", [(64, 16), (96, 24), (128, 128)])
def test_rope_strided(d, rot):
    torch.manual_seed(0)
    s, b, h = 33, 2, 4
    qkv = torch.randn(s, b, h, 3 * d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    q = qkv[..., d:2 * d]                    # a strided view, as sliced from the fused projection
    t = torch.arange(s, device=DEV).float()
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2, device=DEV).float() / rot))
    emb = torch.cat([torch.outer(t, inv)] * 2, dim=-1)
    cos, sin = emb.cos()[:, None, None, :], emb.sin()[:, None, None, :]
    y = OF.rope(q, cos, sin)
    g = torch.randn_like(y)
    y.backward(g)
    qr = qkv.detach().float().requires_grad_()
    yr = OF.rope_ref(qr[..., d:2 * d], cos, sin)
    yr.backward(g.float())
    _close(y, yr, 3e-2)
    _close(qkv.grad, qr.grad, 3e-2)


@pytest.mark.parametrize("dtype,d,rot", [(torch.float32, 64, 64), (torch.float32, 80, 20), (torch.float32, 66, 6),
                                         (torch.float16, 96, 24), (torch.float16, 128, 64), (torch.float16, 80, 20)])
def test_rope_every_vector_width(dtype, d, rot):
    """16-byte, 8-byte and scalar accesses (chosen from rot / 2, d - rot and the strides) give the same rotation."""
    torch.manual_seed(0)
    s, b, h = 17, 3, 5
    x = torch.randn(s, b, h, d, device=DEV, dtype=dtype, requires_grad=True)
    t = torch.arange(s, device=DEV).float()
    inv = 1.0 / (10000 ** (torch.arange(0, rot, 2, device=DEV).float() / rot))
    emb = torch.cat([torch.outer(t, inv)] * 2, dim=-1)
    cos, sin = emb.cos()[:, None, None, :], emb.sin()[:, None, None, :]
    y = OF.rope(x, cos, sin)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_()
    yr = OF.rope_ref(xr, cos, sin)
    yr.backward(g.float())
    tol = 1e-5 if dtype == torch.float32 else 4e-3
    _close(y, yr, tol)
    _close(x.grad, xr.grad, tol)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_cross_entropy(dtype):
    from gpt_neox_b200.parallel.cross_entropy import vocab_parallel_cross_entropy
    torch.manual_seed(0)
    logits = (torch.randn(4, 9, 1000, device=DEV) * 3).to(dtype).requires_grad_()
    tgt = torch.randint(0, 1000, (4, 9), device=DEV)
    loss = vocab_parallel_cross_entropy(logits, tgt)
    w = torch.rand_like(loss)
    (loss * w).sum().backward()
    lr = logits.detach().float().requires_grad_()
    ref = OF.cross_entropy_ref(lr, tgt)
    (ref * w).sum().backward()
    _close(loss, ref, 2e-3 if dtype == torch.float32 else 2e-2)
    _close(logits.grad, lr.grad, 1e-4 if dtype == torch.float32 else 1e-2)


def test_fused_adam_matches_torch():
    from gpt_neox_b200.optim.fused_adam import FusedAdam
    torch.manual_seed(0)
    p0 = torch.randn(10007, device=DEV)
    p1 = torch.nn.Parameter(p0.clone())
    p2 = torch.nn.Parameter(p0.clone())
    out = torch.empty(10007, device=DEV, dtype=torch.bfloat16)
    p1.model_out = out
    o1 = FusedAdam([p1], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    o2 = torch.optim.AdamW([p2], lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    for _ in range(5):
        g = torch.randn(10007, device=DEV)
        p1.grad, p2.grad = g.clone(), g.clone()
        o1.step()
        o2.step()
    _close(p1, p2, 1e-5, rtol=1e-5)
    _close(out, p2, 1e-2)


def test_bounded_wait_reports_instead_of_hanging():
    """A device-side wait that nobody satisfies gives up after its cycle limit, records a status code the host can
    read, and leaves the context usable: a flag-wait kernel is pointed at a flag word that stays 0 (it waits for
    epoch 7 of a second rank that does not exist), on one GPU.  A clean launch before and after reads status 0."""
    import ctypes
    a = torch.randn(128, 64, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(256, 64, device=DEV, dtype=torch.bfloat16)
    G.gemm(a, b)
    assert native.read_status() == 0
    flags = torch.zeros(64, dtype=torch.int32, device=DEV)
    rc = native.lib().neox_wait_flags(native.ptr(flags), ctypes.c_uint(7), 2, 0,
                                      ctypes.c_void_p(native.stream_ptr()))
    assert rc == 0
    assert native.read_status() == 561            # 560 + the rank whose flag never arrived
    out = G.gemm(a, b)                            # the context is intact: kernels still run and are correct
    _close(out, G.gemm_ref(a, b, out_dtype=torch.float32), atol=0.5)
    assert native.read_status() == 0


@pytest.mark.parametrize("sq,sk,b,hq,hkv,d,causal,window,alibi,fused", [
    (128, 128, 1, 1, 1, 64, True, None, False, False),
    (256, 256, 2, 4, 4, 96, True, None, False, True),
    (300, 300, 2, 4, 2, 64, True, None, False, False),      # GQA + ragged tiles
    (200, 200, 1, 2, 2, 128, False, None, False, False),
    (77, 500, 1, 2, 1, 96, True, None, False, False),       # sq < sk: bottom-right aligned causal mask
    (512, 512, 1, 2, 2, 64, True, 100, False, False),       # sliding window
    (512, 512, 1, 2, 2, 64, True, None, True, False),       # ALiBi
    (1024, 1024, 1, 4, 4, 96, True, None, False, True),
])
def test_flash_attention_fwd_bwd(sq, sk, b, hq, hkv, d, causal, window, alibi, fused):
    from gpt_neox_b200.ops import attention as A
    torch.manual_seed(0)
    if fused and hq == hkv:
        qkv = torch.randn(sq, b, hq, 3 * d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        q, k, v = qkv[..., :d], qkv[..., d:2 * d], qkv[..., 2 * d:]
        leaves = [qkv]
    else:
        q = torch.randn(sq, b, hq, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        k = torch.randn(sk, b, hkv, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        v = torch.randn(sk, b, hkv, d, device=DEV, dtype=torch.bfloat16, requires_grad=True)
        leaves = [q, k, v]
    slopes = (torch.rand(hq, device=DEV) * 0.1) if alibi else None
    assert A.have_flash_kernel()
    out = A.flash_attention(q, k, v, causal=causal, window=window, alibi_slopes=slopes)
    g = torch.randn_like(out)
    out.backward(g)
    assert native.read_status() == 0
    refl = [l.detach().float().requires_grad_() for l in leaves]
    if len(refl) == 1:
        rq, rk, rv = refl[0][..., :d], refl[0][..., d:2 * d], refl[0][..., 2 * d:]
    else:
        rq, rk, rv = refl
    ref = A.attention_ref(rq, rk, rv, causal, None, window, slopes)
    ref.backward(g.float())
    _close(out, ref, 3e-2)
    for got, want in zip(leaves, refl):
        _close(got.grad, want.grad, 0.02 + 0.02 * want.grad.abs().max().item(), rtol=3e-2)


@pytest.mark.parametrize("s,b,h,d,rot", [(256, 2, 4, 96, 24), (300, 1, 2, 64, 64), (512, 1, 2, 128, 0)])
def test_packed_qkv_attention_with_inplace_rotary(s, b, h, d, rot):
    """rotary + attention on the packed projection, in place, against fp32 rotary + fp32 attention."""
    from gpt_neox_b200.models.positional import RotaryEmbedding
    from gpt_neox_b200.ops import attention as A
    from gpt_neox_b200.ops import functional as OF
    torch.manual_seed(0)
    mixed = torch.randn(s, b, h, 3 * d, device=DEV, dtype=torch.bfloat16)
    leaf = mixed.clone().requires_grad_(True)
    cos = sin = None
    if rot:
        cos, sin = RotaryEmbedding(rot, s, precision=torch.bfloat16).to(DEV)(mixed, seq_len=s)
    work = leaf * 1.0                                   # non-leaf copy: the op overwrites its input
    out = A.packed_qkv_attention(work, cos, sin)
    g = torch.randn_like(out)
    out.backward(g)
    assert native.read_status() == 0
    ref_leaf = mixed.detach().float().requires_grad_(True)
    q, k, v = ref_leaf[..., :d], ref_leaf[..., d:2 * d], ref_leaf[..., 2 * d:]
    if rot:
        q, k = OF.rope_ref(q, cos, sin), OF.rope_ref(k, cos, sin)
    ref = A.attention_ref(q, k, v, True, None, None, None)
    ref.backward(g.float())
    _close(out, ref, 3e-2)
    _close(leaf.grad, ref_leaf.grad, 0.02 + 0.02 * ref_leaf.grad.abs().max().item(), rtol=3e-2)


def test_flash_attention_is_deterministic():
    from gpt_neox_b200.ops import attention as A
    torch.manual_seed(0)
    q, k, v = (torch.randn(512, 2, 4, 96, device=DEV, dtype=torch.bfloat16, requires_grad=True) for _ in range(3))
    outs, grads = [], []
    for _ in range(2):
        for t in (q, k, v):
            t.grad = None
        o = A.flash_attention(q, k, v)
        o.backward(torch.ones_like(o))
        outs.append(o.detach().clone())
        grads.append([t.grad.clone() for t in (q, k, v)])
    assert torch.equal(outs[0], outs[1])
    for a, b_ in zip(grads[0], grads[1]):
        assert torch.equal(a, b_)      # no atomics anywhere: bitwise repeatable


@pytest.mark.parametrize("b,l,d", [(2, 70, 192), (1, 256, 100)])
def test_selective_scan_fwd_bwd(b, l, d):
    """Mamba S6 scan kernel (state in registers, 32-step checkpoints) against the step-by-step fp32 recurrence."""
    from gpt_neox_b200.ops import selective_scan as SS
    torch.manual_seed(0)
    n = 16
    mk = lambda *s, scale=1.0: (torch.randn(*s, device=DEV) * scale)
    u = mk(b, l, d).to(torch.bfloat16).requires_grad_(True)
    dt = mk(b, l, d, scale=0.5).to(torch.bfloat16).requires_grad_(True)
    z = mk(b, l, d).to(torch.bfloat16).requires_grad_(True)
    A = (-torch.rand(d, n, device=DEV) * 2 - 0.1).requires_grad_(True)
    B = mk(b, l, n, scale=0.5).requires_grad_(True)
    C = mk(b, l, n, scale=0.5).requires_grad_(True)
    D = mk(d).requires_grad_(True)
    bias = mk(d, scale=0.3).requires_grad_(True)
    leaves = [u, dt, A, B, C, D, z, bias]
    assert SS.have_scan_kernel()
    out = SS.selective_scan(u, dt, A, B, C, D, z, bias)
    g = torch.randn_like(out)
    out.backward(g)
    got = [t.grad.clone() for t in leaves]
    for t in leaves:
        t.grad = None
    ref = SS.selective_scan_ref(u.float(), dt.float(), A, B, C, D, z.float(), bias, True)
    ref.backward(g.float())
    _close(out, ref, 3e-2)
    for have, t in zip(got, leaves):
        _close(have, t.grad, 0.03 + 0.03 * t.grad.abs().max().item(), rtol=5e-2)


def test_embedding_kernels_vocab_parallel_slice():
    from gpt_neox_b200.ops import embedding as E
    torch.manual_seed(0)
    V, h, v0 = 1000, 256, 300
    w = torch.randn(400, h, device=DEV, dtype=torch.bfloat16, requires_grad=True)        # owns rows [300, 700)
    ids = torch.randint(0, V, (4, 33), device=DEV)
    ids[0, :5] = 345                                                                      # duplicates: atomics must add
    out = E.embedding(ids, w, v0)
    ref_w = w.detach().float().requires_grad_(True)
    ref = E.embedding_ref(ids, ref_w, v0)
    assert torch.equal(out.float(), ref)
    g = torch.randn_like(out)
    out.backward(g)
    ref.backward(g.float())
    _close(w.grad, ref_w.grad, 2e-2, rtol=2e-2)
    # with an fp32 main-gradient view the kernel accumulates there and autograd sees no .grad
    w2 = w.detach().clone().requires_grad_(True)
    w2.main_grad = torch.ones(400, h, device=DEV, dtype=torch.float32)
    E.embedding(ids, w2, v0).backward(g)
    assert w2.grad is None
    _close(w2.main_grad, 1.0 + ref_w.grad, 1e-3, rtol=1e-4)


@pytest.mark.parametrize("top_k,top_p", [(5, 0.0), (0, 0.9), (50, 0.5), (1, 0.0), (0, 0.999)])
def test_sampling_filter_matches_sort_based_filter(top_k, top_p):
    from gpt_neox_b200 import text_generation as TG
    torch.manual_seed(0)
    logits = torch.randn(7, 50304, device=DEV) * 3
    got = TG.filter_logits(logits, top_k=top_k, top_p=top_p)
    want = TG.filter_logits(logits.cpu(), top_k=top_k, top_p=top_p).to(DEV)
    kept_g, kept_w = torch.isfinite(got), torch.isfinite(want)
    # the sorted reference accumulates 50k fp32 probabilities in another order, so deep in the tail the boundary may
    # move by a few tokens: the sets must agree up to a negligible probability mass
    probs = torch.softmax(logits.float(), dim=-1)
    assert (probs * (kept_g != kept_w)).sum(dim=-1).max().item() < 1e-3
    if top_p < 0.99:
        assert (kept_g != kept_w).sum(dim=-1).max().item() <= 1
    assert torch.equal(got[kept_g & kept_w], logits[kept_g & kept_w])


@pytest.mark.parametrize("along_rows,e5m2", [(False, False), (True, False), (False, True), (True, True)])
def test_mxfp8_quantise_round_trip_matches_torch_float8(along_rows, e5m2):
    from gpt_neox_b200.ops import mxfp8 as MX
    torch.manual_seed(0)
    x = (torch.randn(200, 176, device=DEV) * torch.logspace(-3, 2, 176, device=DEV)).to(torch.bfloat16)
    x[3, :40] = 0
    got = MX.qdq(x, along_rows, e5m2)
    want = MX.qdq_ref(x, along_rows, e5m2)
    assert torch.equal(got, want)
    q, s = MX.quantize(x, along_rows, e5m2)
    assert torch.equal(MX.dequantize(q, s, along_rows, e5m2), got)
    # error of every element is at most 1/8 of its block's maximum: half an ulp of the top binade, or the
    # saturation of scaled values in (max_fp8, 2 * 2^emax) that the power-of-two scale allows
    blk, _, _ = MX._blocks((got.float() - x.float()).abs(), along_rows)
    ref_blk, _, _ = MX._blocks(x.float().abs(), along_rows)
    assert bool((blk.amax(-1) <= ref_blk.amax(-1) * 0.125 + 1e-30).all())


def test_mxfp8_linear_fwd_bwd_against_fp32_on_quantised_operands():
    from gpt_neox_b200.ops import mxfp8 as MX
    torch.manual_seed(0)
    x = torch.randn(256, 192, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(320, 192, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(320, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    y = MX.mx_linear(x, w, b, hybrid=True, fp8_wgrad=True)
    g = torch.randn_like(y)
    y.backward(g)
    xq, wq = MX.qdq_ref(x.detach(), False), MX.qdq_ref(w.detach(), False)
    _close(y, xq.float() @ wq.float().t() + b.float(), 2e-2, rtol=2e-2)
    gq, wq2 = MX.qdq_ref(g, False, True), MX.qdq_ref(w.detach(), True)
    _close(x.grad, gq.float() @ wq2.float(), 2e-2, rtol=2e-2)
    gq2, xq2 = MX.qdq_ref(g, True, True), MX.qdq_ref(x.detach(), True)
    _close(w.grad, gq2.float().t() @ xq2.float(), 5e-2, rtol=2e-2)
    # and the block-scaled result stays close to the unquantised layer
    ref = x.detach().float() @ w.detach().float().t() + b.detach().float()
    assert ((y.float() - ref).abs().mean() / ref.abs().mean()).item() < 0.05


# ------------------------------------------------------------------ per-tensor fp8 (fp8 tensor cores)
@pytest.mark.parametrize("e5m2", [False, True])
def test_fp8_cast_matches_torch_float8(e5m2):
    from gpt_neox_b200.ops import fp8 as F8
    torch.manual_seed(0)
    x = (torch.randn(203, 176, device=DEV) * torch.logspace(-2, 1, 176, device=DEV)).to(torch.bfloat16)
    got = F8.cast(x, e5m2, margin=1)
    want = F8._cast_ref(x, e5m2, 1, None)
    assert torch.allclose(got.inv, want.inv, rtol=1e-6)
    assert torch.equal(got.q, want.q)
    # delayed scaling: the first cast runs at scale 1 and records the amax, the second uses it
    meta = F8.DelayedMeta(x.device, length=4, e5m2=e5m2)
    meta.update()
    first = F8.cast(x, e5m2, meta=meta)
    assert float(first.inv) == 1.0
    meta.update()
    second = F8.cast(x, e5m2, meta=meta)
    lim = F8.E5M2_MAX if e5m2 else F8.E4M3_MAX
    assert abs(float(second.inv) - float(x.float().abs().max()) / lim) < 1e-6 * float(second.inv) + 1e-12
    assert torch.equal(second.q, F8._cast_ref(x, e5m2, 0, None).q)


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
@pytest.mark.parametrize("a_e5,b_e5", [(False, False), (True, False)])
def test_fp8_gemm_matches_fp32_on_the_same_fp8_operands(a_mn, b_mn, a_e5, b_e5):
    from gpt_neox_b200.ops import fp8 as F8
    from gpt_neox_b200.ops import gemm as G
    torch.manual_seed(1)
    M, N, K = 304, 528, 400               # ragged against the 128 x 256 x 128 tile in every dimension
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = (torch.randn((K, N) if b_mn else (N, K), device=DEV) * 0.1).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    aq, bq = F8.cast(a, a_e5), F8.cast(b, b_e5)
    got = F8.gemm_fp8(aq, bq, a_mn, b_mn, bias=bias, out_dtype=torch.float32)
    want = F8.gemm_fp8_ref(aq, bq, a_mn, b_mn, bias=bias, out_dtype=torch.float32)
    _close(got, want, 2e-3, rtol=1e-3)
    acc = torch.randn(M, N, device=DEV)
    got2 = F8.gemm_fp8(aq, bq, a_mn, b_mn, out=acc.clone(), add=acc)
    _close(got2, F8.gemm_fp8_ref(aq, bq, a_mn, b_mn, out_dtype=torch.float32) + acc, 2e-3, rtol=1e-3)


@pytest.mark.parametrize("recipe", ["current", "delayed"])
def test_fp8_linear_fwd_bwd_tracks_the_bf16_layer(recipe):
    from gpt_neox_b200.ops import fp8 as F8
    torch.manual_seed(2)
    x = torch.randn(512, 384, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = torch.nn.Parameter((torch.randn(640, 384, device=DEV) * 0.05).to(torch.bfloat16))
    b = torch.nn.Parameter(torch.randn(640, device=DEV, dtype=torch.bfloat16))
    g = torch.randn(512, 640, device=DEV, dtype=torch.bfloat16)
    rec = F8.Fp8Recipe(recipe=recipe, history_len=4)
    for _ in range(3 if recipe == "delayed" else 1):     # delayed scaling needs a step to learn its scales
        x.grad = w.grad = b.grad = None
        F8.invalidate_weight_cache()                      # what the engine does after an optimizer step
        y = F8.fp8_linear(x, w, b, rec)
        y.backward(g)
    xr, wr = x.detach().float(), w.detach().float()
    rel = lambda got, want: ((got.float() - want).norm() / want.norm()).item()
    assert rel(y, xr @ wr.t() + b.detach().float()) < 0.05
    assert rel(x.grad, g.float() @ wr) < 0.08
    assert rel(w.grad, g.float().t() @ xr) < 0.08
    _close(b.grad, g.float().sum(0), 0.5, rtol=2e-2)
    # exactness against the quantised operands (forward)
    xq, wq = F8._cast_ref(x.detach(), False, 0, None), F8._cast_ref(w.detach(), False, 0, None)
    if recipe == "current":
        _close(y, xq.dequant() @ wq.dequant().t() + b.detach().float(), 3e-2, rtol=1e-2)


# ------------------------------------------------------------------ CTA-pair GEMM (tcgen05 cta_group::2)
@pytest.mark.parametrize("M,N,K,a_mn,b_mn", [(256, 256, 64, 0, 0), (512, 512, 256, 0, 1), (512, 512, 256, 1, 0),
                                             (640, 264, 136, 1, 1), (1000, 840, 328, 0, 0), (77, 96, 200, 0, 1),
                                             (2304, 1536, 512, 0, 0)])
def test_gemm_cta_pair_kernel_matches_fp32(M, N, K, a_mn, b_mn, monkeypatch):
    from gpt_neox_b200.ops import gemm as G
    monkeypatch.setattr(G, "_PAIR", "1")
    torch.manual_seed(0)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = torch.randn((K, N) if b_mn else (N, K), device=DEV, dtype=torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    add = torch.randn(M, N, device=DEV, dtype=torch.float32)
    got = G.gemm(a, b, a_mn, b_mn, bias=bias, add=add, out_dtype=torch.float32)
    want = G.gemm_ref(a, b, a_mn, b_mn, out_dtype=torch.float32, bias=bias, add=add)
    _close(got, want, 2e-2 * (K ** 0.5) / 8, rtol=1e-3)
    got2, pre = G.gemm(a, b, a_mn, b_mn, bias=bias, act=G.ACT_GELU, want_preact=True)
    want2, wpre = G.gemm_ref(a, b, a_mn, b_mn, bias=bias, act=G.ACT_GELU, want_preact=True)
    _close(pre, wpre, 0.25, rtol=1e-2)
    _close(got2, want2, 0.25, rtol=1e-2)
    from gpt_neox_b200.ops import native
    assert native.read_status() == 0


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, False), (True, True)])
def test_fp8_gemm_cta_pair_kernel_matches_fp32_on_the_same_fp8_operands(a_mn, b_mn, monkeypatch):
    from gpt_neox_b200.ops import fp8 as F8
    from gpt_neox_b200.ops import gemm as G
    from gpt_neox_b200.ops import native
    monkeypatch.setattr(G, "_PAIR", "1")
    torch.manual_seed(1)
    M, N, K = 560, 528, 400
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = (torch.randn((K, N) if b_mn else (N, K), device=DEV) * 0.1).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    aq, bq = F8.cast(a, True), F8.cast(b, False)
    got = F8.gemm_fp8(aq, bq, a_mn, b_mn, bias=bias, out_dtype=torch.float32)
    want = F8.gemm_fp8_ref(aq, bq, a_mn, b_mn, bias=bias, out_dtype=torch.float32)
    _close(got, want, 2e-3, rtol=1e-3)
    assert native.read_status() == 0


# ------------------------------------------------------------------ MXFP8 on the block-scaled tensor cores
@pytest.mark.parametrize("a_rows,b_rows", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("mode", ["unit_scales", "row_scales", "k_scales", "random"])
def test_mxfp8_block_scaled_gemm_matches_dequantised_product(a_rows, b_rows, mode):
    """forward (K-major, K-major), dgrad (K-major, MN-major) and wgrad (MN-major, MN-major) layouts; the scale
    patterns isolate the scale plumbing: all scales equal / varying along mn only / along K blocks only / both."""
    from gpt_neox_b200.ops import mxfp8 as MX
    from gpt_neox_b200.ops import gemm as G
    torch.manual_seed(3)
    M, N, K = 272, 464, 416          # N: three 192-wide tiles (even, odd, ragged); K: ragged against 128
    def make(mn, k, rows_are_k):
        base = torch.empty(mn, k, device=DEV).uniform_(1.0, 1.9)
        sign = torch.where(torch.rand(mn, k, device=DEV) < 0.5, -1.0, 1.0)
        mn_e = torch.randint(-3, 4, (mn, 1), device=DEV).float()
        k_e = torch.randint(-3, 4, (1, (k + 31) // 32), device=DEV).float().repeat_interleave(32, dim=1)[:, :k]
        e = {"unit_scales": 0 * mn_e + 0 * k_e, "row_scales": mn_e + 0 * k_e, "k_scales": 0 * mn_e + k_e,
             "random": mn_e + k_e}[mode]
        t = (base * sign * torch.exp2(e)).to(torch.bfloat16)          # [mn, k]
        return t.t().contiguous() if rows_are_k else t
    a = make(M, K, a_rows)           # [M, K] or [K, M]
    b = make(N, K, b_rows)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    got = MX.gemm_mx(MX.quantize_tiled(a, a_rows, False), MX.quantize_tiled(b, b_rows, True), bias=bias,
                     out_dtype=torch.float32)
    want = G.gemm_ref(MX.qdq_ref(a, a_rows, False), MX.qdq_ref(b, b_rows, True), a_rows, b_rows,
                      out_dtype=torch.float32, bias=bias)
    assert native.read_status() == 0
    _close(got, want, 1e-2, rtol=2e-3)


def test_mxfp8_hardware_linear_matches_the_emulated_layer():
    from gpt_neox_b200.ops import mxfp8 as MX
    torch.manual_seed(0)
    x = torch.randn(256, 192, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(320, 192, device=DEV) * 0.05).to(torch.bfloat16).requires_grad_(True)
    b = torch.randn(320, device=DEV, dtype=torch.bfloat16, requires_grad=True)
    g = torch.randn(256, 320, device=DEV, dtype=torch.bfloat16)
    outs = []
    for hw in (False, True):
        x.grad = w.grad = b.grad = None
        y = MX.mx_linear(x, w, b, hybrid=True, fp8_wgrad=True, hardware=hw)
        y.backward(g)
        outs.append((y.detach().float(), x.grad.float().clone(), w.grad.float().clone()))
    for e, h in zip(*outs):
        _close(h, e, 3e-2, rtol=2e-2)


@pytest.mark.parametrize("e5m2", [False, True])
def test_mxfp8_dual_quantise_equals_the_two_single_direction_passes(e5m2):
    from gpt_neox_b200.ops import mxfp8 as MX
    torch.manual_seed(5)
    x = (torch.randn(203, 2184, device=DEV) * torch.logspace(-3, 2, 2184, device=DEV)).to(torch.bfloat16)
    x[40:80, 64:96] = 0
    tc, tr = MX.quantize_dual(x, e5m2)
    sc, sr = MX.quantize_tiled(x, False, e5m2), MX.quantize_tiled(x, True, e5m2)
    assert torch.equal(tc.q, sc.q) and torch.equal(tc.sf, sc.sf) and tc.mnb == sc.mnb
    assert torch.equal(tr.q, sr.q) and torch.equal(tr.sf, sr.sf) and tr.mnb == sr.mnb


# ------------------------------------------------------------------ fp16 operands, long persistent loops, small kernels
@pytest.mark.parametrize("pair", ["0", "1"])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_fp16_operands(a_mn, b_mn, pair, monkeypatch):
    """fp16 A / B / bias / output through both tcgen05 kernels (instruction-descriptor format bit + fp16 epilogue)."""
    monkeypatch.setattr(G, "_PAIR", pair)
    torch.manual_seed(0)
    M, N, K = 520, 776, 392
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.float16)
    b = (torch.randn((K, N) if b_mn else (N, K), device=DEV) * 0.1).to(torch.float16)
    bias = torch.randn(N, device=DEV, dtype=torch.float16)
    res = torch.randn(M, N, device=DEV, dtype=torch.float16)
    got, pre = G.gemm(a, b, a_mn, b_mn, bias=bias, act=G.ACT_GELU, add=res, want_preact=True)
    assert got.dtype == torch.float16 and pre.dtype == torch.float16
    want, wpre = G.gemm_ref(a, b, a_mn, b_mn, bias=bias, act=G.ACT_GELU, add=res, want_preact=True, out_dtype=torch.float32)
    _close(pre, wpre, 0.02, rtol=4e-3)           # fp16 keeps 11 bits: tighter than the bf16 cases above
    _close(got, want, 0.02, rtol=4e-3)
    acc = torch.randn(M, N, device=DEV, dtype=torch.float32)
    want = G.gemm_ref(a, b, a_mn, b_mn, add=acc, out_dtype=torch.float32)
    G.gemm(a, b, a_mn, b_mn, out=acc, add=acc)
    _close(acc, want, 0.02, rtol=2e-3)
    assert native.read_status() == 0


@pytest.mark.parametrize("pair", ["0", "1"])
@pytest.mark.parametrize("M,N,K", [(4096, 4096, 512), (8192, 6144, 1024)])
@pytest.mark.parametrize("a_mn,b_mn", [(0, 0), (0, 1), (1, 0), (1, 1)])
def test_gemm_many_tiles_per_cta(M, N, K, a_mn, b_mn, pair, monkeypatch):
    """Problems with several tiles per persistent CTA (accumulator double-buffering, barrier phase flips over many
    tiles, L2 tile order) against the fp32 product."""
    monkeypatch.setattr(G, "_PAIR", pair)
    torch.manual_seed(2)
    a = torch.randn((K, M) if a_mn else (M, K), device=DEV, dtype=torch.bfloat16)
    b = (torch.randn((K, N) if b_mn else (N, K), device=DEV) * 0.05).to(torch.bfloat16)
    bias = torch.randn(N, device=DEV, dtype=torch.bfloat16)
    got = G.gemm(a, b, a_mn, b_mn, bias=bias, out_dtype=torch.float32)
    want = G.gemm_ref(a, b, a_mn, b_mn, bias=bias, out_dtype=torch.float32)
    _close(got, want, 0.03, rtol=2e-3)
    assert native.read_status() == 0


@pytest.mark.parametrize("sq,sk,b,hq,hkv,d,causal", [(256, 256, 2, 4, 4, 96, True), (300, 300, 1, 4, 2, 64, True),
                                                     (200, 328, 1, 2, 2, 128, False)])
def test_flash_attention_fp16(sq, sk, b, hq, hkv, d, causal):
    from gpt_neox_b200.ops import attention as A
    torch.manual_seed(0)
    q = torch.randn(sq, b, hq, d, device=DEV, dtype=torch.float16, requires_grad=True)
    k = torch.randn(sk, b, hkv, d, device=DEV, dtype=torch.float16, requires_grad=True)
    v = torch.randn(sk, b, hkv, d, device=DEV, dtype=torch.float16, requires_grad=True)
    out = A.flash_attention(q, k, v, causal=causal)
    assert out.dtype == torch.float16
    g = torch.randn_like(out)
    out.backward(g)
    assert native.read_status() == 0
    refl = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = A.attention_ref(*refl, causal, None, None, None)
    ref.backward(g.float())
    _close(out, ref, 1e-2)
    for got, want in zip((q, k, v), refl):
        _close(got.grad, want.grad, 0.01 + 0.01 * want.grad.abs().max().item(), rtol=1e-2)


@pytest.mark.parametrize("B,T,H,N", [(2, 64, 4, 64), (1, 100, 2, 64)])
def test_wkv6_kernel_matches_reference_scan(B, T, H, N):
    """RWKV-6 wkv forward and backward (CUDA) against the sequential fp32 recurrence."""
    from gpt_neox_b200.ops import wkv6 as W
    torch.manual_seed(0)
    C = H * N
    mk = lambda scale=1.0: (torch.randn(B, T, C, device=DEV) * scale).to(torch.bfloat16).requires_grad_()
    r, k, v = mk(), mk(0.5), mk()
    w = (-torch.rand(B, T, C, device=DEV) * 2 - 0.1).to(torch.bfloat16).requires_grad_()      # log-decay, negative
    u = (torch.randn(H, N, device=DEV) * 0.3).to(torch.bfloat16).requires_grad_()
    y = W.wkv6(r, k, v, w, u)
    g = torch.randn_like(y)
    y.backward(g)
    got = [t.grad.clone() for t in (r, k, v, w, u)]
    ref_in = [t.detach().float().requires_grad_() for t in (r, k, v, w, u)]
    yr = W.wkv6_ref(*ref_in)
    yr.backward(g.float())
    _close(y, yr, 0.05 + 0.02 * yr.abs().max().item(), rtol=2e-2)
    for a, b_ in zip(got, ref_in):
        _close(a, b_.grad, 0.05 + 0.03 * b_.grad.abs().max().item(), rtol=3e-2)


def test_lion_kernel_matches_eager_update():
    from gpt_neox_b200.optim.lion import Lion
    torch.manual_seed(0)
    n = 100_003
    p0 = torch.randn(n, device=DEV)
    grads = [torch.randn(n, device=DEV) for _ in range(3)]
    p_gpu = torch.nn.Parameter(p0.clone())
    out = torch.empty(n, device=DEV, dtype=torch.bfloat16)
    p_gpu.model_out = out
    p_cpu = torch.nn.Parameter(p0.cpu().clone())
    o_gpu = Lion([p_gpu], lr=1e-2, betas=(0.9, 0.98), weight_decay=0.1)
    o_cpu = Lion([p_cpu], lr=1e-2, betas=(0.9, 0.98), weight_decay=0.1)
    for g in grads:
        p_gpu.grad, p_cpu.grad = g.clone(), g.cpu().clone()
        o_gpu.step()
        o_cpu.step()
    # a sign flip needs |m*b1 + g*(1-b1)| at rounding level: allow a handful of elements to differ by 2*lr
    diff = (p_gpu.detach().cpu() - p_cpu.detach()).abs()
    assert (diff > 1e-5).sum().item() <= 3, diff.max()
    _close(out, p_gpu.detach(), 1e-2, rtol=1e-2)
    _close(o_gpu.state[p_gpu]["exp_avg"].cpu(), o_cpu.state[p_cpu]["exp_avg"], 1e-5, rtol=1e-4)


def test_adam8bit_tracks_fp32_adam():
    """Block-wise 8-bit optimizer states: after 20 steps on a quadratic the parameters stay close to fp32 Adam."""
    from gpt_neox_b200.optim.adam8bit import Adam8bit
    torch.manual_seed(0)
    n = 4096 + 77
    target = torch.randn(n, device=DEV)
    p8 = torch.nn.Parameter(torch.zeros(n, device=DEV))
    p32 = torch.nn.Parameter(torch.zeros(n, device=DEV))
    o8 = Adam8bit([p8], lr=5e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.0)
    o32 = torch.optim.Adam([p32], lr=5e-2, betas=(0.9, 0.95), eps=1e-8)
    for _ in range(20):
        for p, o in ((p8, o8), (p32, o32)):
            p.grad = (p.detach() - target) * (1 + 0.1 * torch.randn(n, device=DEV, generator=None))
            o.step()
    assert (p8 - p32).abs().max().item() < 0.15 and (p8 - target).norm() < 0.8 * target.norm()
    st = o8.state[p8]
    assert any(t.dtype in (torch.int8, torch.uint8) for t in st.values() if torch.is_tensor(t))
    # the CUDA kernel and the chunked torch statement of the same update agree (same quantised states, same result)
    pc = torch.nn.Parameter(torch.zeros(n))
    oc = Adam8bit([pc], lr=5e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    pg = torch.nn.Parameter(torch.zeros(n, device=DEV))
    og = Adam8bit([pg], lr=5e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    gen = torch.Generator().manual_seed(5)
    for _ in range(5):
        gr = torch.randn(n, generator=gen)
        pc.grad, pg.grad = gr.clone(), gr.to(DEV)
        oc.step()
        og.step()
    _close(pg.detach().cpu(), pc.detach(), 2e-3, rtol=1e-3)
    assert (og.state[pg]["qm"].cpu().int() - oc.state[pc]["qm"].int()).abs().max().item() <= 1
    # the 16-bit model copy written by the same kernel is the rounded fp32 parameter, tail block included
    pm = torch.nn.Parameter(torch.zeros(n, device=DEV))
    pm.model_out = torch.full((n,), 7.0, device=DEV, dtype=torch.bfloat16)
    om = Adam8bit([pm], lr=5e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.01)
    for _ in range(3):
        pm.grad = torch.randn(n, device=DEV)
        om.step()
    assert torch.equal(pm.model_out, pm.detach().bfloat16())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float32])
def test_bias_dropout_add_kernel_matches_the_philox_mask(dtype):
    """Training-mode bias + dropout + residual add in one kernel: forward and backward against the same Philox
    mask generated in plain torch; the keep rate is 1 - p; a replayed generator state reproduces the mask."""
    torch.manual_seed(123)
    rows, cols, p = 300, 1024, 0.1
    x = torch.randn(rows, cols, device=DEV, dtype=dtype, requires_grad=True)
    bias = torch.randn(cols, device=DEV, dtype=dtype, requires_grad=True)
    res = torch.randn(rows, cols, device=DEV, dtype=dtype, requires_grad=True)
    gen = torch.cuda.default_generators[torch.cuda.current_device()]
    state = torch.cuda.get_rng_state()
    seed, offset = gen.initial_seed(), gen.get_offset()
    out = OF.bias_dropout_add(x, bias, res, p, True)
    assert gen.get_offset() > offset                       # the stream was advanced: the next call draws a new mask
    keep = OF.philox_mask_ref(rows * cols, p, seed, offset, device=DEV).view(rows, cols)
    assert abs(keep.float().mean().item() - (1 - p)) < 5e-3
    want = res.float() + torch.where(keep, (x.float() + bias.float()) / (1 - p), torch.zeros((), device=DEV))
    _close(out, want, 2e-2 if dtype != torch.float32 else 1e-5)
    g = torch.randn_like(out)
    out.backward(g)
    gx = torch.where(keep, g.float() / (1 - p), torch.zeros((), device=DEV))
    _close(x.grad, gx, 2e-2 if dtype != torch.float32 else 1e-5)
    _close(res.grad, g, 0.0, rtol=0.0)
    _close(bias.grad, gx.sum(0), 0.5 if dtype != torch.float32 else 1e-3, rtol=2e-2)
    torch.cuda.set_rng_state(state)                        # what activation checkpointing does before recomputing
    again = OF.bias_dropout_add(x.detach(), bias.detach(), res.detach(), p, True)
    assert torch.equal(again, out.detach())
    other = OF.bias_dropout_add(x.detach(), bias.detach(), res.detach(), p, True)
    assert not torch.equal(other, out.detach())


# ------------------------------------------------------------------ mixture-of-experts kernels
@pytest.mark.parametrize("T,E,k,dtype", [(1000, 8, 2, torch.bfloat16), (513, 64, 1, torch.float32),
                                         (300, 200, 4, torch.float16)])
def test_moe_router_kernel_matches_eager(T, E, k, dtype):
    from gpt_neox_b200.ops import moe_ops as MO
    torch.manual_seed(0)
    logits = (torch.randn(T, E, device=DEV) * 2).to(dtype)
    a = logits.clone().requires_grad_(True)
    b = logits.clone().requires_grad_(True)
    probs, w, idx, counts = MO.router(a, k)
    probs_r, w_r, idx_r, counts_r = MO.router_ref(b, k)
    _close(probs, probs_r, 1e-6, rtol=1e-4)
    _close(w, w_r, 1e-6, rtol=1e-4)
    # ties between equal probabilities (frequent with 16-bit logits) may be broken differently: the selected
    # probabilities always agree; indices, histogram and gradients are compared on the rows without a tie
    assert torch.equal(probs_r.gather(1, idx).sort(1).values, probs_r.gather(1, idx_r).sort(1).values)
    rows = (idx == idx_r).all(1)
    assert rows.float().mean().item() > 0.9
    if bool(rows.all()):
        assert torch.equal(counts, counts_r)
    assert int(counts.sum()) == T * k
    gw = torch.randn(T, k, device=DEV)
    gp = torch.randn(T, E, device=DEV) * 0.1
    (w * gw).sum().add((probs * gp).sum()).backward()
    (w_r * gw).sum().add((probs_r * gp).sum()).backward()
    lo = dtype != torch.float32
    _close(a.grad[rows], b.grad[rows], 4e-3 if lo else 1e-5, rtol=2e-2 if lo else 1e-3)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_moe_dispatch_and_combine_kernels(dtype):
    from gpt_neox_b200.ops import moe_ops as MO
    torch.manual_seed(1)
    T, E, k, h = 700, 8, 2, 264
    idx = torch.stack([torch.randperm(E, device=DEV)[:k] for _ in range(T)])
    counts = torch.bincount(idx.reshape(-1), minlength=E)
    for cap in (None, 100):
        row_of, kept = MO.plan_rows(idx, counts, cap)
        rows = MO.padded_rows(T * k, E)
        # every kept assignment has its own row inside its expert's segment
        flat = row_of.reshape(-1)
        ok = flat >= 0
        assert flat[ok].unique().numel() == int(ok.sum()) == int(kept.sum())
        starts = torch.cumsum((kept + 63) // 64 * 64, 0) - (kept + 63) // 64 * 64
        e_of = idx.reshape(-1)[ok]
        assert bool(((flat[ok] >= starts[e_of]) & (flat[ok] < starts[e_of] + kept[e_of])).all())
        x = torch.randn(T, h, device=DEV).to(dtype)
        gate = torch.rand(T, k, device=DEV)
        xa = x.clone().requires_grad_(True)
        xb = x.clone().requires_grad_(True)
        ga = gate.clone().requires_grad_(True)
        gb = gate.clone().requires_grad_(True)
        pa = MO.dispatch(xa, row_of, rows)
        pb = MO.dispatch_ref(xb, row_of, rows)
        assert torch.equal(pa, pb)
        ya = MO.combine(pa * 1.0, row_of, ga)
        yb = MO.combine_ref(pb * 1.0, row_of, gb)
        _close(ya, yb, 1e-2)
        gy = torch.randn_like(ya)
        ya.backward(gy)
        yb.backward(gy)
        _close(xa.grad, xb.grad, 2e-2)
        _close(ga.grad, gb.grad, 5e-2, rtol=2e-2)


@pytest.mark.parametrize("counts,N,K,act", [([300, 0, 129, 64, 1, 700, 5, 90], 512, 256, None),
                                            ([37, 1000], 384, 192, "gelu"),
                                            ([0, 0, 0, 256], 256, 64, "gelu")])
def test_grouped_gemm_matches_per_expert_eager(counts, N, K, act):
    from gpt_neox_b200.ops import moe_ops as MO
    torch.manual_seed(2)
    E = len(counts)
    cnt = torch.tensor(counts, device=DEV)
    rows = MO.padded_rows(sum(counts), E)
    x = torch.zeros(rows, K, device=DEV, dtype=torch.bfloat16)
    g = torch.zeros(rows, N, device=DEV, dtype=torch.bfloat16)
    row = 0
    for c in counts:
        x[row:row + c] = torch.randn(c, K, device=DEV).to(torch.bfloat16)
        g[row:row + c] = torch.randn(c, N, device=DEV).to(torch.bfloat16)
        row += (c + 63) // 64 * 64
    w = (torch.randn(E, N, K, device=DEV) / math.sqrt(K)).to(torch.bfloat16)
    assert MO.grouped_kernel_ok(x, w)
    xa, wa = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    xb, wb = x.float().requires_grad_(True), w.float().requires_grad_(True)
    ya = MO.grouped_linear(xa, wa, cnt, act)
    yb = MO.grouped_linear_ref(xb, wb, cnt, act)
    assert native.read_status() == 0
    _close(ya, yb, 3e-2, rtol=2e-2)
    ya.backward(g)
    yb.backward(g.float())
    assert native.read_status() == 0
    _close(xa.grad, xb.grad, 5e-2, rtol=3e-2)
    _close(wa.grad, wb.grad, 0.25, rtol=3e-2)
    # weight gradients accumulate into the optimizer's fp32 buffer when it is attached
    wa2 = w.clone().requires_grad_(True)
    wa2.main_grad = torch.ones(E, N, K, device=DEV)
    MO.grouped_linear(x.clone().requires_grad_(True), wa2, cnt, act).backward(g)
    _close(wa2.main_grad - 1.0, wb.grad, 0.25, rtol=3e-2)


@pytest.mark.parametrize("rows,cols,dtype", [(4096, 6144, torch.bfloat16), (1000, 264, torch.float16), (7, 8, torch.bfloat16)])
def test_bias_grad_column_sum_kernel(rows, cols, dtype):
    torch.manual_seed(3)
    g = torch.randn(rows, cols, device=DEV).to(dtype)
    ref = g.float().sum(0)
    out = OF.bias_grad(g)
    assert out.dtype == dtype
    _close(out, ref, 0.05 * math.sqrt(rows) / 8, rtol=1e-2)
    # with the optimizer's fp32 buffer attached the sum is accumulated there and the parameter is reported ready
    bias = torch.nn.Parameter(torch.zeros(cols, device=DEV, dtype=dtype))
    bias.main_grad = torch.full((cols,), 2.0, device=DEV)
    seen = []
    bias._grad_ready = lambda: seen.append(1)
    assert OF.bias_grad(g, bias) is None and seen == [1] and bias.grad_in_main
    _close(bias.main_grad - 2.0, ref, 1e-3 * math.sqrt(rows), rtol=1e-5)
    # a strided view (the rows of a wider matrix)
    wide = torch.randn(rows, cols * 2, device=DEV).to(dtype)
    _close(OF.bias_grad(wide[:, :cols]), wide[:, :cols].float().sum(0), 0.05 * math.sqrt(rows) / 8, rtol=1e-2)


@pytest.mark.parametrize("kinds", [("ln", "ln"), ("ln",), ("rms",), ("rms", "ln")])
def test_norm_fan_out_adds_all_gradient_contributions_in_the_kernels(kinds):
    """Block head ``x -> (norms(x)..., x)``: outputs equal the separate norm kernels bit for bit; the input gradient is
    the sum of the residual gradient and every norm's gradient (fp32 oracle); parameter gradients as usual."""
    from gpt_neox_b200.models.norms import LayerNorm, RMSNorm
    torch.manual_seed(4)
    rows, b, h = 192, 3, 1024
    mods = [LayerNorm(h, eps=1e-5, device=DEV, dtype=torch.bfloat16) if k == "ln"
            else RMSNorm(h, eps=1e-6, device=DEV, dtype=torch.bfloat16) for k in kinds]
    for m in mods:
        for p in m.parameters():
            p.data.add_(torch.randn_like(p) * 0.2)
    x = torch.randn(rows, b, h, device=DEV).to(torch.bfloat16)
    gs = [torch.randn(rows, b, h, device=DEV).to(torch.bfloat16) for _ in range(len(mods) + 1)]
    xa = x.clone().requires_grad_(True)
    outs = OF.norm_fan_out(xa, mods)
    assert len(outs) == len(mods) + 1 and outs[-1].data_ptr() == xa.data_ptr()
    sep = [m(x) for m in mods]
    for o, s in zip(outs, sep):
        assert torch.equal(o, s)
    torch.autograd.backward(list(outs), gs)
    got = {id(p): p.grad.clone() for m in mods for p in m.parameters()}
    for m in mods:
        m.zero_grad()
    # fp32 oracle through the modules' eager math
    xb = x.float().requires_grad_(True)
    ws = [p for m in mods for p in m.parameters()]
    wf = [p.detach().float().requires_grad_(True) for p in ws]
    ref_outs = []
    it = iter(wf)
    for m, k in zip(mods, kinds):
        if k == "ln":
            w_, b_ = next(it), next(it)
            ref_outs.append(torch.nn.functional.layer_norm(xb, (h,), w_, b_, m.eps))
        else:
            s_ = next(it)
            ref_outs.append(xb / (xb.norm(2, dim=-1, keepdim=True) * h ** -0.5 + m.eps) * s_)
    torch.autograd.backward(ref_outs + [xb * 1.0], [g.float() for g in gs])
    _close(xa.grad, xb.grad, 0.06, rtol=2e-2)
    for p, f in zip(ws, wf):
        _close(got[id(p)], f.grad, 0.02 * math.sqrt(rows * b), rtol=3e-2)
    # only some outputs used: the others contribute nothing (no zero tensors are materialised for them)
    xc = x.clone().requires_grad_(True)
    outs = OF.norm_fan_out(xc, mods)
    outs[0].backward(gs[0])
    xd = x.clone().requires_grad_(True)
    mods[0](xd).backward(gs[0])
    _close(xc.grad, xd.grad, 1e-6, rtol=0)


def test_block_sparse_attention_on_device_bf16():
    from gpt_neox_b200.models.transformer import sparse_layout_mask
    from gpt_neox_b200.ops.sparse_attention import block_sparse_attention
    torch.manual_seed(0)
    s, b, h, d = 1000, 2, 8, 64
    cfg = {"block": 16, "num_sliding_window_blocks": 5, "num_global_blocks": 2, "num_random_blocks": 2}
    q, k, v = [torch.randn(s, b, h, d, device=DEV).to(torch.bfloat16).requires_grad_(True) for _ in range(3)]
    out = block_sparse_attention(q, k, v, "bigbird", cfg, d ** -0.5)
    g = torch.randn_like(out)
    out.backward(g)
    mask = sparse_layout_mask("bigbird", s, s, cfg, q.device) | \
        (torch.arange(s, device=DEV)[None, :] > torch.arange(s, device=DEV)[:, None])
    qf, kf, vf = [t.detach().float().requires_grad_(True) for t in (q, k, v)]
    probs = torch.softmax((torch.einsum("sbhd,tbhd->bhst", qf, kf) * d ** -0.5).masked_fill(mask[None, None],
                                                                                           float("-inf")), dim=-1)
    ref = torch.einsum("bhst,tbhd->sbhd", probs, vf)
    ref.backward(g.float())
    _close(out, ref, 2e-2, rtol=2e-2)
    for a, r in ((q.grad, qf.grad), (k.grad, kf.grad), (v.grad, vf.grad)):
        _close(a, r, 6e-2, rtol=5e-2)


@pytest.mark.parametrize("n,offset", [(1, 0), (7, 1), (1000003, 0), (1000003, 3), (4096, 2)])
def test_squared_norm_kernel_any_alignment(n, offset):
    import ctypes
    torch.manual_seed(6)
    base = torch.randn(n + offset + 8, device=DEV)
    x = base[offset:offset + n]
    out = torch.zeros((), device=DEV)
    rc = native.lib().neox_sumsq_f32(native.ptr(x), ctypes.c_longlong(n), native.ptr(out),
                                     ctypes.c_void_p(native.stream_ptr()))
    native.check(rc, "neox_sumsq_f32")
    ref = (x.double() ** 2).sum().item()
    assert abs(out.item() - ref) <= 2e-5 * max(ref, 1.0), (out.item(), ref)
