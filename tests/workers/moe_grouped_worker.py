"""One GPU: the mixture-of-experts layer with the fused router / dispatch / grouped-GEMM / combine kernels against
the per-expert loop over the plain GEMM (same weights, same input): outputs and all gradients agree to bf16 accuracy,
then a small MoE model trains with the grouped path (the loss falls)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from common import make_args  # noqa: E402


def main():
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models.init_functions import get_init_methods
    from gpt_neox_b200.models.moe import ParallelMoE
    from gpt_neox_b200.ops import native
    from gpt_neox_b200.training import setup_model_and_optimizer, train_step
    from gpt_neox_b200.utils import Timers
    cfg = dict(hidden_size=256, num_attention_heads=4, moe_num_experts=8, moe_top_k=2, precision="bfloat16",
               distributed_backend="nccl", seq_length=512, max_position_embeddings=512, expert_interval=1,
               gpt_j_residual=False, train_micro_batch_size_per_gpu=4)
    args = make_args(**cfg)
    args.configure_distributed_args()
    initialize_megatron(args)
    init, out_init = get_init_methods(args)
    for extra in ({}, {"moe_token_dropping": True, "moe_train_capacity_factor": 0.75}):
        for k, v in extra.items():
            setattr(args, k, v)
        moe = ParallelMoE(args, init, out_init, 8)
        x = torch.randn(512, 4, 256, device="cuda").to(torch.bfloat16)
        assert moe._use_grouped(x.view(-1, 256))
        res = []
        for grouped in (False, None):
            moe.grouped = grouped
            moe.zero_grad()
            xi = x.clone().requires_grad_(True)
            y, lbl = moe(xi)
            (y.float().square().sum() + lbl.float()).backward()
            res.append((y.detach(), xi.grad, moe.w1.grad.clone(), moe.w2.grad.clone(),
                        moe.router.layer.weight.grad.clone()))
        assert native.read_status() == 0
        for name, a, b in zip(("y", "dx", "dw1", "dw2", "drouter"), *res):
            a, b = a.float(), b.float()
            err = (a - b).abs().max().item()
            scale = b.abs().max().item()
            assert err <= 0.04 * max(scale, 1e-3), (name, err, scale)
    args = make_args(**cfg)
    args.configure_distributed_args()
    model, opt, sched, _ = setup_model_and_optimizer(args)
    g = torch.Generator().manual_seed(0)
    batches = [{"text": torch.randint(0, args.padded_vocab_size, (4, args.seq_length + 1), generator=g)}
               for _ in range(2)]

    def it():
        i = 0
        while True:
            yield batches[i % 2]
            i += 1
    data = it()
    losses = [float(train_step(args, Timers(), data, model, opt, sched)[0]["lm_loss"]) for _ in range(12)]
    assert native.read_status() == 0
    assert min(losses[6:]) < losses[0] - 0.3, losses
    print("MOE_GROUPED_OK", losses[0], losses[-1], flush=True)


if __name__ == "__main__":
    main()
