#!/usr/bin/env python
"""Import a Hugging Face GPT-NeoX or Llama-family model into the native sequential checkpoint layout
(``mp_rank_XX_model_states.pt`` with ``sequential.{idx}.{name}`` keys), sharded for a tensor-parallel degree.

    python -m gpt_neox_b200.tools.ckpts.convert_hf_to_sequential --hf_model <dir-or-name> --output_dir ckpts/imported \\
        --model_parallel_size 2 [--architecture neox|llama]

Inverse of the merge rules: column-parallel tensors are split along dim 0, row-parallel weights along dim 1,
norms are replicated and row-parallel biases are divided by the tensor-parallel degree (each rank adds its share
before the deferred reduction of the parallel-residual block).  Llama q/k/v are re-packed into the fused QKV
layout the model uses (per-head interleaved for MHA, ``[Q|K|V]`` for GQA) and ``[up ; gate]`` for the gated MLP.
"""
from __future__ import annotations

import argparse
import os

import torch


def shard(t, mp, dim):
    return list(torch.chunk(t, mp, dim=dim))


def convert(hf_model, mp=1, architecture="neox"):
    """Returns ``[state_dict_rank0, ...]`` with sequential keys."""
    sd = hf_model.state_dict()
    cfg = hf_model.config
    L, heads = cfg.num_hidden_layers, cfg.num_attention_heads
    hd = cfg.hidden_size // heads
    out = [dict() for _ in range(mp)]

    def put(idx, name, tensors):
        for r in range(mp):
            out[r][f"sequential.{idx}.{name}"] = tensors[r].clone().contiguous()

    rep = lambda t: [t] * mp
    if architecture == "neox":
        put(0, "word_embeddings.weight", shard(sd["gpt_neox.embed_in.weight"], mp, 0))
        for i in range(L):
            p = f"gpt_neox.layers.{i}."
            put(i + 2, "attention.query_key_value.weight", shard(sd[p + "attention.query_key_value.weight"], mp, 0))
            put(i + 2, "attention.dense.weight", shard(sd[p + "attention.dense.weight"], mp, 1))
            put(i + 2, "mlp.linear1.weight", shard(sd[p + "mlp.dense_h_to_4h.weight"], mp, 0))
            put(i + 2, "mlp.linear2.weight", shard(sd[p + "mlp.dense_4h_to_h.weight"], mp, 1))
            for k, nk in (("attention.query_key_value.bias", "attention.query_key_value.bias"),
                          ("mlp.dense_h_to_4h.bias", "mlp.linear1.bias")):
                if p + k in sd:
                    put(i + 2, nk, shard(sd[p + k], mp, 0))
            for k, nk in (("attention.dense.bias", "attention.dense.bias"), ("mlp.dense_4h_to_h.bias", "mlp.linear2.bias")):
                if p + k in sd:
                    put(i + 2, nk, rep(sd[p + k] / mp))
            for k in ("input_layernorm.weight", "input_layernorm.bias", "post_attention_layernorm.weight",
                      "post_attention_layernorm.bias"):
                put(i + 2, k, rep(sd[p + k]))
        put(L + 3, "norm.weight", rep(sd["gpt_neox.final_layer_norm.weight"]))
        put(L + 3, "norm.bias", rep(sd["gpt_neox.final_layer_norm.bias"]))
        put(L + 4, "final_linear.weight", shard(sd["embed_out.weight"], mp, 0))
    else:
        kvh = getattr(cfg, "num_key_value_heads", heads) or heads
        put(0, "word_embeddings.weight", shard(sd["model.embed_tokens.weight"], mp, 0))
        for i in range(L):
            p = f"model.layers.{i}."
            q, k, v = sd[p + "self_attn.q_proj.weight"], sd[p + "self_attn.k_proj.weight"], sd[p + "self_attn.v_proj.weight"]
            fused = []
            for r in range(mp):
                if kvh == heads:
                    n = heads // mp
                    qq = q.view(heads, hd, -1)[r * n:(r + 1) * n]
                    kk = k.view(heads, hd, -1)[r * n:(r + 1) * n]
                    vv = v.view(heads, hd, -1)[r * n:(r + 1) * n]
                    fused.append(torch.stack([qq, kk, vv], dim=1).reshape(n * 3 * hd, -1))
                else:
                    nq, nk = heads // mp * hd, kvh // mp * hd
                    fused.append(torch.cat([q[r * nq:(r + 1) * nq], k[r * nk:(r + 1) * nk], v[r * nk:(r + 1) * nk]], 0))
            put(i + 2, "attention.query_key_value.weight", fused)
            put(i + 2, "attention.dense.weight", shard(sd[p + "self_attn.o_proj.weight"], mp, 1))
            ups, gates = shard(sd[p + "mlp.up_proj.weight"], mp, 0), shard(sd[p + "mlp.gate_proj.weight"], mp, 0)
            put(i + 2, "mlp.linear1.weight", [torch.cat([u, g], 0) for u, g in zip(ups, gates)])
            put(i + 2, "mlp.linear2.weight", shard(sd[p + "mlp.down_proj.weight"], mp, 1))
            put(i + 2, "input_layernorm.scale", rep(sd[p + "input_layernorm.weight"]))
            put(i + 2, "post_attention_layernorm.scale", rep(sd[p + "post_attention_layernorm.weight"]))
        put(L + 3, "norm.scale", rep(sd["model.norm.weight"]))
        put(L + 4, "final_linear.weight", shard(sd["lm_head.weight"], mp, 0))
    return out


def save(shards, output_dir, tag="global_step0"):
    d = os.path.join(output_dir, tag)
    os.makedirs(d, exist_ok=True)
    for r, sd in enumerate(shards):
        torch.save({"module": sd, "optimizer": None, "lr_scheduler": None, "dp_world_size": 1, "mp_world_size": len(shards),
                    "global_steps": 0, "global_samples": 0, "skipped_steps": 0, "iteration": 0},
                   os.path.join(d, f"mp_rank_{r:02d}_model_states.pt"))
    with open(os.path.join(output_dir, "latest"), "w") as fh:
        fh.write(tag)


def main(argv=None):
    from transformers import AutoModelForCausalLM
    ap = argparse.ArgumentParser()
    ap.add_argument("--hf_model", required=True)
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--model_parallel_size", type=int, default=1)
    ap.add_argument("--architecture", default="neox", choices=["neox", "llama", "mistral"])
    a = ap.parse_args(argv)
    hf = AutoModelForCausalLM.from_pretrained(a.hf_model)
    save(convert(hf, a.model_parallel_size, "neox" if a.architecture == "neox" else "llama"), a.output_dir)
    print(f"wrote {a.model_parallel_size} shard(s) to {a.output_dir}")


if __name__ == "__main__":
    main()
