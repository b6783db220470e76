"""Operator-level checks that run on CPU (eager statements of the kernels' math)."""
import pytest
import torch




def test_fp8_linear_gelu_split_matches_plain_composition():
    """fc1 (GeLU, split pre-activation) -> fc2 (GeLU' folded into dgrad) in fp8 gives the gradients of the plain
    composition ``fc2(gelu(fc1(x)))`` evaluated on the same quantised operands' math (loose: fp8 rounding)."""
    import torch
    from gpt_neox_b200.ops import fp8 as F8
    torch.manual_seed(0)
    x = torch.randn(64, 32).bfloat16().requires_grad_(True)
    w1 = torch.nn.Parameter((torch.randn(48, 32) * 0.2).bfloat16())
    w2 = torch.nn.Parameter((torch.randn(32, 48) * 0.2).bfloat16())
    rec = F8.Fp8Recipe(hybrid=False)
    h, pre = F8.fp8_linear(x, w1, None, rec, act="gelu", split_pre=True)
    y = F8.fp8_linear(h, w2, None, rec, residual=x, dgelu_aux=pre)
    y.float().pow(2).sum().backward()
    got = [t.grad.float().clone() for t in (x, w1, w2)]
    for t in (x, w1, w2):
        t.grad = None
    yr = torch.nn.functional.gelu(x.float() @ w1.float().t(), approximate="tanh") @ w2.float().t() + x.float()
    yr.pow(2).sum().backward()
    assert ((y.float() - yr).norm() / yr.norm()).item() < 0.05
    for g, t in zip(got, (x, w1, w2)):
        assert ((g - t.grad.float()).norm() / t.grad.float().norm()).item() < 0.12


def test_fp8_delayed_scaling_history_and_weight_cache():
    import torch
    from gpt_neox_b200.ops import fp8 as F8
    m = F8.DelayedMeta(torch.device("cpu"), length=3, e5m2=False, margin=1, most_recent=False)
    m.update()
    assert float(m.buf[0]) == 1.0 and float(m.buf[1]) == 1.0            # nothing seen yet: scale 1
    x = torch.tensor([[0.5, -2.0], [1.0, 0.25]]).bfloat16()
    F8.cast(x, meta=m)
    assert float(m.buf[2]) == 2.0                                        # recorded amax
    m.update()
    assert abs(float(m.buf[0]) - 448.0 / (2.0 * 2.0)) < 1e-6             # fp8_max / (amax * 2^margin)
    F8.cast(x * 0.25, meta=m)
    m.update()
    assert abs(float(m.buf[0]) - 448.0 / (2.0 * 2.0)) < 1e-6             # 'max' over the history keeps the larger amax
    mr = F8.DelayedMeta(torch.device("cpu"), length=3, most_recent=True)
    mr.update(); F8.cast(x, meta=mr); mr.update(); F8.cast(x * 0.25, meta=mr); mr.update()
    assert abs(float(mr.buf[0]) - 448.0 / 0.5) < 1e-4                    # 'most_recent' follows the last amax

    w = torch.nn.Parameter(torch.randn(16, 16).bfloat16())
    rec = F8.Fp8Recipe()
    a = F8._cast_weight(w, rec)
    assert F8._cast_weight(w, rec) is a                                  # cached
    F8.invalidate_weight_cache()
    assert F8._cast_weight(w, rec) is not a                              # the engine's optimizer step invalidates
    with torch.no_grad():
        w.add_(1.0)                                                      # so does an in-place update autograd can see
    b = F8._cast_weight(w, rec)
    assert not torch.equal(b.q, a.q)


def test_pair_kernel_selection(monkeypatch):
    from gpt_neox_b200.ops import gemm as G
    monkeypatch.setattr(G, "_PAIR", "auto")
    assert G.use_pair_kernel(8192, 6144, 6144)                           # fills the machine with 256 x 256 tiles
    assert not G.use_pair_kernel(512, 512, 4096)                         # 4 tiles: one-CTA kernel
    assert not G.use_pair_kernel(8192, 6144, 128)                        # short K: nothing to pipeline
    monkeypatch.setattr(G, "_PAIR", "0")
    assert not G.use_pair_kernel(8192, 6144, 6144)
    monkeypatch.setattr(G, "_PAIR", "1")
    assert G.use_pair_kernel(64, 64, 64)


@pytest.mark.parametrize("kind,cfg", [
    ("local", {"block": 16, "num_sliding_window_blocks": 3}),
    ("sparse_fixed", {"block": 8, "num_local_blocks": 4, "num_global_blocks": 1}),
    ("sparse_variable", {"block": 16, "num_local_blocks": 2}),
    ("bigbird", {"block": 16, "num_sliding_window_blocks": 3, "num_global_blocks": 1, "num_random_blocks": 2}),
    ("bslongformer", {"block": 16, "num_sliding_window_blocks": 3, "global_block_indices": [0, 2]}),
])
def test_block_sparse_attention_matches_the_dense_masked_statement(kind, cfg):
    """Gathering only the kept tiles gives the same output and gradients as masking a dense score matrix."""
    from gpt_neox_b200.models.transformer import sparse_layout_mask
    from gpt_neox_b200.ops.sparse_attention import block_sparse_attention
    torch.manual_seed(0)
    s, b, h, hkv, d = 100, 2, 4, 2, 8                      # s is not a multiple of the block; grouped-query heads
    q = torch.randn(s, b, h, d, requires_grad=True)
    k = torch.randn(s, b, hkv, d, requires_grad=True)
    v = torch.randn(s, b, hkv, d, requires_grad=True)
    scale = d ** -0.5
    out = block_sparse_attention(q, k, v, kind, cfg, scale)
    g = torch.randn_like(out)
    out.backward(g)
    got = (out.detach(), q.grad.clone(), k.grad.clone(), v.grad.clone())
    for t in (q, k, v):
        t.grad = None
    mask = sparse_layout_mask(kind, s, s, cfg, q.device) | (torch.arange(s)[None, :] > torch.arange(s)[:, None])
    kf = k.repeat_interleave(h // hkv, dim=2)
    vf = v.repeat_interleave(h // hkv, dim=2)
    scores = torch.einsum("sbhd,tbhd->bhst", q, kf) * scale
    probs = torch.softmax(scores.masked_fill(mask[None, None], float("-inf")), dim=-1)
    ref = torch.einsum("bhst,tbhd->sbhd", probs, vf)
    ref.backward(g)
    for a, r in zip(got, (ref.detach(), q.grad, k.grad, v.grad)):
        torch.testing.assert_close(a, r, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("adamw", [True, False])
def test_cpu_adam_host_kernel_matches_torch(adamw):
    """The OpenMP / AVX2 host kernel against torch's Adam / AdamW: host parameters are updated in place, the bf16
    copy is the rounded parameter, a gradient scale is folded in."""
    from gpt_neox_b200.optim.cpu_adam import CPUAdam
    torch.manual_seed(0)
    n = 1000 + 37
    p = torch.nn.Parameter(torch.randn(n))
    q = torch.nn.Parameter(p.detach().clone())
    p.model_out = torch.zeros(n, dtype=torch.bfloat16)
    kw = dict(lr=1e-2, betas=(0.9, 0.95), eps=1e-8, weight_decay=0.1)
    ours = CPUAdam([p], adamw_mode=adamw, **kw)
    ref = (torch.optim.AdamW if adamw else torch.optim.Adam)([q], **kw)
    ours.param_groups[0]["grad_scale"] = 0.5
    storage = p.data_ptr()
    for _ in range(5):
        g = torch.randn(n)
        p.grad, q.grad = g * 2.0, g.clone()               # the scale of 0.5 undoes the factor
        ours.step()
        ref.step()
    assert p.data_ptr() == storage and "host_param" not in ours.state[p]
    torch.testing.assert_close(p.detach(), q.detach(), atol=2e-6, rtol=1e-5)
    assert torch.equal(p.model_out, p.detach().bfloat16())
