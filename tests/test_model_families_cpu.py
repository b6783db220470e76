"""Every mixer family builds and trains on CPU: MoE (dropless and capacity), RWKV-6, Mamba, gMLP/aMLP,
sparse-attention layouts; plus operator oracles for wkv6 and the selective scan."""
import pytest
import torch

from common import run_distributed
from test_training_cpu import _loss_decreases


@pytest.mark.parametrize("cfg", [
    {"moe_num_experts": 4, "moe_top_k": 2, "expert_interval": 1, "moe_token_dropping": False, "gpt_j_residual": False},
    {"moe_num_experts": 4, "moe_top_k": 1, "expert_interval": 2, "moe_token_dropping": True,
     "moe_train_capacity_factor": 1.25, "gpt_j_residual": False},
    # DeepSpeed-style MoE: a dense MLP beside the experts, mixed by a learned per-token coefficient
    {"moe_num_experts": 4, "moe_top_k": 1, "expert_interval": 1, "moe_type": "deepspeed", "moe_use_residual": True,
     "moe_token_dropping": True, "gpt_j_residual": False},
    {"attention_config": [[["rwkv"], "all"]], "num_attention_heads": 2, "hidden_size": 64, "pos_emb": "none"},
    {"attention_config": [[["mamba"], "all"]], "pos_emb": "none"},
    {"attention_config": [[["gmlp"], 1], [["amlp"], 1]], "pos_emb": "none", "gpt_j_residual": False},
    {"attention_config": [[["global", "bigbird"], 1]], "sparsity_config": {"block": 4}},
    {"attention_config": [[["local", "bslongformer"], 1]], "sparsity_config": {"block": 4}},
    {"sliding_window_width": 8},
    # block-scaled fp8 linears (the Transformer-Engine switches of the 1-3B-transformer-engine config)
    {"te_columnparallel": True, "te_rowparallel": True, "te_fp8_format": "hybrid", "precision": "bfloat16"},
    {"te_columnparallel": True, "te_rowparallel": True, "te_fp8_recipe": "delayed", "te_fp8_amax_history_len": 4,
     "te_fp8_amax_compute_algo": "max", "precision": "bfloat16"},
    {"te_columnparallel": True, "te_rowparallel": True, "te_fp8_recipe": "mxfp8", "precision": "bfloat16"},
    {"te_rowparallel": True, "precision": "bfloat16"},        # bf16 fc1 hands its pre-activation to an fp8 fc2
])
def test_family_trains(cfg):
    run_distributed(_loss_decreases, 1, cfg, None)


def test_moe_expert_parallel_two_ranks():
    run_distributed(_loss_decreases, 2, {"moe_num_experts": 4, "moe_top_k": 2, "expert_interval": 1,
                                         "moe_expert_parallel_size": 2, "gpt_j_residual": False}, None)


def _ep4_loop_vs_grouped(rank, world):
    """Four expert-parallel ranks with two local experts each: with few tokens many (source rank, expert) segments
    are empty, which the receive-side bookkeeping has to survive; the per-expert loop and the grouped form give the
    same training."""
    import torch
    from test_training_cpu import _setup, _train
    from gpt_neox_b200.models.moe import ParallelMoE
    from gpt_neox_b200.parallel import mpu
    runs = []
    for grouped in (False, True):
        torch.manual_seed(0)
        args, model, opt, sched = _setup({"global_num_gpus": world, "moe_num_experts": 8, "moe_top_k": 2,
                                          "expert_interval": 2, "moe_expert_parallel_size": 4,
                                          "gpt_j_residual": False, "moe_token_dropping": False})
        moes = [m for m in model.module.modules() if isinstance(m, ParallelMoE)]
        assert moes and all(m.ep == 4 and m.local_experts == 2 for m in moes)
        for m in moes:
            m.grouped = grouped
        runs.append(_train(args, model, opt, sched, 8))
        mpu.destroy_model_parallel()
    assert min(runs[0]) < runs[0][0]
    for a, b in zip(*runs):
        assert abs(a - b) < 1e-4, runs


def test_moe_expert_parallel_four_ranks_two_local_experts():
    run_distributed(_ep4_loop_vs_grouped, 4)


def test_wkv6_reference_gradients_are_consistent():
    """The closed form used for the decay gradient (reverse cumulative sums of r*grS and k*gkG) equals autograd
    through the plain recurrence."""
    from gpt_neox_b200.ops.wkv6 import wkv6_ref
    torch.manual_seed(0)
    B, T, H, N = 2, 7, 2, 4
    C = H * N
    r, k, v = (torch.randn(B, T, C, dtype=torch.float64, requires_grad=True) for _ in range(3))
    w = (torch.randn(B, T, C, dtype=torch.float64) * 0.5 - 1).requires_grad_()
    u = torch.randn(H, N, dtype=torch.float64, requires_grad=True)
    gy = torch.randn(B, T, C, dtype=torch.float64)

    def f64(r, k, v, w, u):
        rf, kf, vf = (t.view(B, T, H, N) for t in (r, k, v))
        d = torch.exp(-torch.exp(w)).view(B, T, H, N)
        S = torch.zeros(B, H, N, N, dtype=torch.float64)
        ys, states = [], []
        for t in range(T):
            states.append(S)
            kv = kf[:, t, :, :, None] * vf[:, t, :, None, :]
            ys.append(torch.einsum("bhj,bhji->bhi", rf[:, t], u[None, :, :, None] * kv + S))
            S = S * d[:, t, :, :, None] + kv
        return torch.stack(ys, 1).reshape(B, T, C), states

    y, states = f64(r, k, v, w, u)
    y.backward(gy)
    # re-derive gw with the scalar identity from per-step quantities
    rf, kf, vf, gyf = (t.detach().view(B, T, H, N) for t in (r, k, v, gy))
    d = torch.exp(-torch.exp(w.detach())).view(B, T, H, N)
    grS = torch.stack([torch.einsum("bhji,bhi->bhj", states[t].detach(), gyf[:, t]) for t in range(T)], 1)
    G = torch.zeros(B, H, N, N, dtype=torch.float64)
    gkG = [None] * T
    for t in reversed(range(T)):
        gkG[t] = torch.einsum("bhi,bhji->bhj", vf[:, t], G)
        G = G * d[:, t, :, :, None] + rf[:, t, :, :, None] * gyf[:, t, :, None, :]
    gkG = torch.stack(gkG, 1)
    a, b = rf * grS, kf * gkG
    ra = torch.flip(torch.cumsum(torch.flip(a, [1]), 1), [1]) - a
    rb = torch.flip(torch.cumsum(torch.flip(b, [1]), 1), [1])
    gw = ((ra - rb) * (-torch.exp(w.detach())).view(B, T, H, N)).reshape(B, T, C)
    assert torch.allclose(gw, w.grad, atol=1e-9), (gw - w.grad).abs().max()
    assert torch.allclose(wkv6_ref(r.detach().float(), k.detach().float(), v.detach().float(), w.detach().float(),
                                   u.detach().float()).double(), y.detach(), atol=1e-4)


def _moe_grouped_matches_loop(rank, world, cfg):
    """The grouped data flow (router -> row plan -> dispatch -> grouped linears -> combine) against the per-expert
    loop: same outputs, same gradients, with and without a capacity limit."""
    import torch
    from common import make_args
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models.init_functions import get_init_methods
    from gpt_neox_b200.models.moe import ParallelMoE
    args = make_args(**{**cfg, "global_num_gpus": world})
    args.configure_distributed_args()
    initialize_megatron(args)
    init, out_init = get_init_methods(args)
    moe = ParallelMoE(args, init, out_init, args.moe_num_experts).float()
    x = torch.randn(args.seq_length, 3, args.hidden_size)
    res = []
    for grouped in (False, True):
        moe.grouped = grouped
        moe.zero_grad()
        xi = x.clone().requires_grad_(True)
        y, lbl = moe(xi)
        (y.square().sum() + lbl).backward()
        res.append((y.detach(), lbl.detach(), xi.grad, moe.w1.grad.clone(), moe.w2.grad.clone(),
                    moe.router.layer.weight.grad.clone()))
    for a, b in zip(*res):
        torch.testing.assert_close(a, b, atol=2e-5, rtol=1e-4)


@pytest.mark.parametrize("cfg", [
    {"moe_num_experts": 4, "moe_top_k": 2, "moe_token_dropping": False},
    {"moe_num_experts": 8, "moe_top_k": 1, "moe_token_dropping": True, "moe_train_capacity_factor": 0.5,
     "moe_min_capacity": 2},
    {"moe_num_experts": 4, "moe_top_k": 2, "moe_token_dropping": False, "moe_glu": True, "activation": "swiglu"},
])
def test_moe_grouped_data_flow_matches_per_expert_loop(cfg):
    run_distributed(_moe_grouped_matches_loop, 1, cfg)


def _moe_capacity_edges(rank, world):
    """``moe_min_capacity`` is a floor under the capacity formula; assignments beyond an expert's capacity are
    dropped in token order; a token with every assignment dropped contributes nothing (and gets no gradient)."""
    import torch
    from common import make_args
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models.init_functions import get_init_methods
    from gpt_neox_b200.models.moe import ParallelMoE
    from gpt_neox_b200.ops import moe_ops as MO
    args = make_args(global_num_gpus=world, moe_num_experts=8, moe_top_k=1, moe_token_dropping=True,
                     moe_train_capacity_factor=0.01, moe_eval_capacity_factor=2.0, moe_min_capacity=3)
    args.configure_distributed_args()
    initialize_megatron(args)
    init, out_init = get_init_methods(args)
    moe = ParallelMoE(args, init, out_init, 8).float()
    moe.train()
    assert moe._capacity(16) == 3                      # ceil(0.01 * 16 / 8) = 1 < the floor
    assert moe._capacity(100000) == 125                # the formula once it exceeds the floor
    moe.eval()
    assert moe._capacity(16) == 4                      # the evaluation factor: ceil(2.0 * 16 / 8)
    moe.train()

    idx = torch.tensor([[0], [0], [1], [0], [0], [0], [1]])
    counts = torch.bincount(idx.reshape(-1), minlength=8)
    row_of, kept = MO.plan_rows(idx, counts, capacity=3)
    assert kept.tolist() == [3, 2, 0, 0, 0, 0, 0, 0]
    assert row_of.reshape(-1).tolist() == [0, 1, MO.PAD, 2, -1, -1, MO.PAD + 1]      # tokens 4 and 5 overflow expert 0

    # route every token to expert 0: only the first three survive
    with torch.no_grad():
        moe.router.layer.weight.zero_()
        moe.router.layer.weight[0].fill_(1.0)
    x = torch.rand(6, 1, args.hidden_size) + 0.5       # positive features: expert 0 has the largest logit
    for grouped in (False, True):
        moe.grouped = grouped
        xi = x.clone().requires_grad_(True)
        y, _ = moe(xi)
        assert bool((y[3:] == 0).all()) and bool((y[:3].abs().sum(-1) > 0).all())
        y.sum().backward()
        assert bool((xi.grad[3:] == 0).all())


def test_moe_min_capacity_and_overflow():
    run_distributed(_moe_capacity_edges, 1)


def _expert_tensor_parallel(rank, world):
    """Experts sharded over the tensor-parallel group against a dense statement with the full weights: outputs,
    input gradient, router gradient (replicated) and expert-weight gradients (the matching slices) agree."""
    import torch
    import torch.distributed as dist
    import torch.nn.functional as F
    from common import make_args
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models.init_functions import get_init_methods
    from gpt_neox_b200.models.moe import ParallelMoE
    from gpt_neox_b200.parallel import mpu
    args = make_args(global_num_gpus=world, model_parallel_size=world, moe_num_experts=4, moe_top_k=2,
                     moe_token_dropping=False, enable_expert_tensor_parallelism=True)
    args.configure_distributed_args()
    initialize_megatron(args)
    init, out_init = get_init_methods(args)
    moe = ParallelMoE(args, init, out_init, 4).float()
    assert moe.expert_tp and moe.w1.shape[1] == 4 * args.hidden_size // world and moe.w1.model_parallel
    grp = mpu.get_model_parallel_group()

    def gather(t, dim):
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous(), group=grp)
        return torch.cat(parts, dim=dim)

    W1 = gather(moe.w1.detach(), 1).requires_grad_(True)
    W2 = gather(moe.w2.detach(), 2).requires_grad_(True)
    Wr = moe.router.layer.weight.detach().clone().requires_grad_(True)
    torch.manual_seed(5)
    x = torch.randn(args.seq_length, 2, args.hidden_size)
    xa = x.clone().requires_grad_(True)
    y, lbl = moe(xa)
    (y.square().sum() + lbl).backward()
    xb = x.clone().requires_grad_(True)
    flat = xb.reshape(-1, args.hidden_size)
    probs = F.softmax(flat @ Wr.t(), dim=-1)
    w, idx = torch.topk(probs, 2, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    ref = torch.zeros_like(flat)
    for e in range(4):
        gate = (w * (idx == e)).sum(-1, keepdim=True)
        ref = ref + gate * (F.gelu(flat @ W1[e].t(), approximate="tanh") @ W2[e].t())
    counts = torch.bincount(idx.reshape(-1), minlength=4).float()
    lbl_ref = 4 * torch.sum(counts / counts.sum() * probs.mean(0))
    (ref.square().sum() + lbl_ref).backward()
    tol = dict(atol=3e-5, rtol=1e-4)
    torch.testing.assert_close(y.reshape(-1, args.hidden_size), ref, **tol)
    torch.testing.assert_close(xa.grad, xb.grad, **tol)
    torch.testing.assert_close(moe.router.layer.weight.grad, Wr.grad, **tol)
    f = moe.ffn
    torch.testing.assert_close(moe.w1.grad, W1.grad[:, rank * f:(rank + 1) * f], **tol)
    torch.testing.assert_close(moe.w2.grad, W2.grad[:, :, rank * f:(rank + 1) * f], **tol)


def test_moe_expert_tensor_parallelism_matches_dense_math():
    run_distributed(_expert_tensor_parallel, 2)
