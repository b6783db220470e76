

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
