"""2-GPU expert-parallel MoE block: peer-memory token exchange against the NCCL all-to-all (launched by torchrun).
Prints ``MOE_A2A_OK`` on rank 0 when outputs and gradients of both paths agree on every rank."""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))


def main():
    from common import make_args
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.models.init_functions import get_init_methods
    from gpt_neox_b200.models.moe import ParallelMoE
    from gpt_neox_b200.ops import native
    from gpt_neox_b200.parallel import moe_comm
    world = int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
    args = make_args(hidden_size=256, num_attention_heads=4, precision="bfloat16", global_num_gpus=world,
                     distributed_backend="nccl", moe_num_experts=4, moe_top_k=2, moe_expert_parallel_size=world,
                     expert_interval=1, gpt_j_residual=False, moe_token_dropping=False)
    args.configure_distributed_args()
    initialize_megatron(args)
    init, out_init = get_init_methods(args)
    torch.manual_seed(99)
    moe = ParallelMoE(args, init, out_init, 4)
    dev = torch.device("cuda", torch.cuda.current_device())
    g = torch.Generator(device=dev).manual_seed(5 + dist.get_rank())
    ok = True
    for it in range(4):                                   # several exchanges: both buffer parities are reused
        x = torch.randn(48 + 16 * it, 2, 256, device=dev, generator=g).to(torch.bfloat16)
        gy = torch.randn(48 + 16 * it, 2, 256, device=dev, generator=g).to(torch.bfloat16)
        res = {}
        for mode, comb in (("1", "1"), ("1", "0"), ("0", "0")):
            os.environ["NEOX_FUSED_MOE_A2A"] = mode
            os.environ["NEOX_FUSED_MOE_COMBINE"] = comb
            mode = mode + comb
            for p in moe.parameters():
                p.grad = None
            xi = x.clone().requires_grad_(True)
            y, aux = moe(xi)
            (y.float() * gy.float()).sum().backward()
            res[mode] = [y.detach(), xi.grad] + [p.grad.clone() for p in moe.parameters()]
        for variant in ("11", "10"):
            for i, (a, b) in enumerate(zip(res[variant], res["00"])):
                err = (a.float() - b.float()).abs().max().item()
                if err > 1e-2 * (b.float().abs().max().item() + 1e-6):
                    print(f"[rank {dist.get_rank()}] it {it} variant {variant} tensor {i}: max err {err}", flush=True)
                    ok = False
    if native.read_status() != 0:
        ok = False
    flag = torch.tensor([int(ok)], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if dist.get_rank() == 0 and flag.item() == 1:
        print("MOE_A2A_OK", flush=True)
    dist.barrier()
    moe_comm.reset()
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
