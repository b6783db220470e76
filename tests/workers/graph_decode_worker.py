"""One GPU: token-by-token decoding replayed from a CUDA graph (fixed-capacity key/value caches) against the ordinary
growing-cache decoding of the same bf16 model: the per-step logits agree to bf16 accuracy, the graph was captured once
and replayed for every later token, and the replayed step is faster than the eager one."""
import os
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from common import make_args  # noqa: E402


def main():
    from gpt_neox_b200 import text_generation as TG
    from gpt_neox_b200.initialize import initialize_megatron
    from gpt_neox_b200.training import setup_model_and_optimizer
    args = make_args(hidden_size=512, num_attention_heads=8, num_layers=6, seq_length=256, max_position_embeddings=256,
                     precision="bfloat16", distributed_backend="nccl", optimizer=None, no_load_optim=True,
                     return_logits=True)
    args.configure_distributed_args()
    initialize_megatron(args)
    model, _, _, _ = setup_model_and_optimizer(args, use_cache=True)
    model.module.inference_mode(use_cache=True)
    # sample 0 is a long prompt: its tokens are forced at every step, so both runs feed it identical inputs and its
    # recorded logits can be compared position by position; sample 1 generates freely from a short prompt
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, 500, (124,), generator=g).tolist(), [9, 10, 11]]
    seen = []
    orig = TG.GraphDecoder.step

    def step(self, *a):
        out = orig(self, *a)
        seen.append((self.graph is not None, self.steps))
        return out
    TG.GraphDecoder.step = step
    res, ms = {}, {}
    for graph in (False, True, False, True):
        args.update_value("cuda_graph_decode", graph)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        last = None
        for last in TG.stream_tokens(args, model, prompts, eos_token_id=-1, maximum_tokens=120):
            pass
        torch.cuda.synchronize()
        ms[graph] = (time.perf_counter() - t0) * 1e3
        res[graph] = (last[0].clone(), last[3].clone())
    assert seen and all(g for g, _ in seen) and max(n for _, n in seen) >= 100, seen[:3]
    a, b = res[False][1][:118], res[True][1][:118]
    err = (a - b).abs().max().item()
    assert err < 0.06 * max(a.abs().max().item(), 1.0), (err, a.abs().max().item())
    assert torch.equal(res[False][0][0], res[True][0][0])
    assert ms[True] < ms[False], ms
    print(f"GRAPH_DECODE_OK eager {ms[False]:.0f} ms, graph {ms[True]:.0f} ms for 120 tokens; max logit difference "
          f"{err:.4f}", flush=True)


if __name__ == "__main__":
    main()
