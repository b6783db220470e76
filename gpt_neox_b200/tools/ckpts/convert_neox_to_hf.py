#!/usr/bin/env python
"""Convert a native checkpoint (sequential ``mp_rank_XX_model_states.pt`` or per-layer
``layer_XX-model_YY-model_states.pt`` files, any tensor-parallel degree) to a Hugging Face model directory.

    python -m gpt_neox_b200.tools.ckpts.convert_neox_to_hf --input_dir ckpt/global_step1000 \\
        --config_file cfg.yml --output_dir hf_out [--architecture neox|llama|mistral] [--precision bf16]

Tensor-parallel merge rules (the same ones every GPT-NeoX tool applies, ``tools/ckpts/convert_neox_to_hf.py:596-648``
of the reference): column-parallel weights and biases are concatenated along dim 0, row-parallel weights along
dim 1, norm parameters are averaged, row-parallel biases are summed.  Layout facts used:
  * fused QKV of multi-head attention is per-head interleaved ``[heads, 3, head_dim]`` -- identical to HF GPT-NeoX;
  * grouped-query QKV is contiguous ``[Q | K | V]`` per rank;
  * gated MLP ``linear1`` holds ``[up ; gate]`` halves per rank -> ``up_proj`` / ``gate_proj``.
"""
from __future__ import annotations

import argparse
import os

import torch
import yaml

MODEL_KEYS = {
    "neox": {
        "COLUMN_PARALLEL_LINEAR_KEYS": {"mlp.linear1.weight": "mlp.dense_h_to_4h.weight", "mlp.linear1.bias": "mlp.dense_h_to_4h.bias",
                                        "attention.query_key_value.weight": "attention.query_key_value.weight",
                                        "attention.query_key_value.bias": "attention.query_key_value.bias"},
        "ROW_PARALLEL_LINEAR_KEYS": {"attention.dense.weight": "attention.dense.weight", "mlp.linear2.weight": "mlp.dense_4h_to_h.weight"},
        "ROW_PARALLEL_BIAS_KEYS": {"mlp.linear2.bias": "mlp.dense_4h_to_h.bias", "attention.dense.bias": "attention.dense.bias"},
        "NORM_KEYS": {"input_layernorm.weight": "input_layernorm.weight", "input_layernorm.bias": "input_layernorm.bias",
                      "post_attention_layernorm.weight": "post_attention_layernorm.weight",
                      "post_attention_layernorm.bias": "post_attention_layernorm.bias"},
        "FINAL_NORM_KEYS": {"norm.weight": "weight", "norm.bias": "bias"},
    },
    "llama": {
        "ROW_PARALLEL_LINEAR_KEYS": {"attention.dense.weight": "self_attn.o_proj.weight", "mlp.linear2.weight": "mlp.down_proj.weight"},
        "ROW_PARALLEL_BIAS_KEYS": {},
        "NORM_KEYS": {"input_layernorm.scale": "input_layernorm.weight", "post_attention_layernorm.scale": "post_attention_layernorm.weight"},
        "FINAL_NORM_KEYS": {"norm.scale": "weight"},
    },
}
MODEL_KEYS["mistral"] = MODEL_KEYS["llama"]


def load_config(path):
    cfg = {}
    for f in ([path] if isinstance(path, str) else path):
        with open(f) as fh:
            cfg.update({k.replace("-", "_"): v for k, v in (yaml.load(fh, Loader=yaml.FullLoader) or {}).items()})
    return cfg


def get_key(cfg, key, default=None):
    v = cfg.get(key, cfg.get(key.replace("_", "-"), None))
    return default if v is None else v


def load_partitions(input_dir, mp, layer_idx, sequential):
    """State dicts of one layer from every tensor-parallel rank (keys without the layer prefix)."""
    if sequential:
        parts = []
        for i in range(mp):
            sd = torch.load(os.path.join(input_dir, f"mp_rank_{i:02d}_model_states.pt"), map_location="cpu",
                            weights_only=False)["module"]
            pre = f"sequential.{layer_idx}."
            parts.append({k[len(pre):]: v for k, v in sd.items() if k.startswith(pre)})
        return parts
    return [torch.load(os.path.join(input_dir, f"layer_{layer_idx:02d}-model_{i:02d}-model_states.pt"),
                       map_location="cpu", weights_only=False) for i in range(mp)]


def get_state(parts, key, layer_idx=None, sequential=None):
    return [p[key] for p in parts]


def create_config(cfg, architecture="neox", pad_token=0):
    from transformers import GPTNeoXConfig, LlamaConfig, MistralConfig
    heads = get_key(cfg, "num_attention_heads")
    hidden = get_key(cfg, "hidden_size")
    common = dict(vocab_size=get_key(cfg, "padded_vocab_size") or get_key(cfg, "vocab_size", 50432), hidden_size=hidden,
                  num_hidden_layers=get_key(cfg, "num_layers"), num_attention_heads=heads,
                  max_position_embeddings=get_key(cfg, "max_position_embeddings"),
                  initializer_range=get_key(cfg, "init_method_std", 0.02),
                  tie_word_embeddings=not get_key(cfg, "no_weight_tying", False), use_cache=True)
    if architecture == "neox":
        inter = get_key(cfg, "intermediate_size") or int(get_key(cfg, "expansion_factor", 4) * hidden)
        return GPTNeoXConfig(**common, intermediate_size=inter, hidden_act="gelu_fast",
                             rotary_pct=get_key(cfg, "rotary_pct", 1.0), rotary_emb_base=get_key(cfg, "rotary_emb_base", 10000),
                             layer_norm_eps=get_key(cfg, "layernorm_epsilon", 1e-5),
                             use_parallel_residual=get_key(cfg, "gpt_j_residual", False), bos_token_id=pad_token,
                             eos_token_id=pad_token, attention_bias=get_key(cfg, "use_bias_in_attn_linear", True))
    from ...models.transformer import mlp_dims
    from types import SimpleNamespace
    ns = SimpleNamespace(intermediate_size=get_key(cfg, "intermediate_size"), expansion_factor=get_key(cfg, "expansion_factor"),
                         hidden_size=hidden, activation=get_key(cfg, "activation", "swiglu"),
                         mlp_multiple_of=get_key(cfg, "mlp_multiple_of", 1))
    _, ffn_in = mlp_dims(ns)
    kw = dict(**common, intermediate_size=ffn_in, hidden_act="silu", rms_norm_eps=get_key(cfg, "rms_norm_epsilon", 1e-6),
              num_key_value_heads=get_key(cfg, "num_kv_heads") or heads, rope_theta=get_key(cfg, "rotary_emb_base", 10000))
    if architecture == "mistral":
        return MistralConfig(**kw, sliding_window=get_key(cfg, "sliding_window_width", 4096))
    return LlamaConfig(**kw)


def convert(input_dir, cfg, output_dir=None, sequential=None, precision=None, architecture="neox"):
    from transformers import AutoModelForCausalLM
    mp = get_key(cfg, "model_parallel_size", 1)
    L = get_key(cfg, "num_layers")
    if sequential is None:
        sequential = os.path.exists(os.path.join(input_dir, "mp_rank_00_model_states.pt")) and \
            not os.path.exists(os.path.join(input_dir, "layer_00-model_00-model_states.pt"))
    hf_config = create_config(cfg, architecture)
    hf = AutoModelForCausalLM.from_config(hf_config)
    if precision:
        hf = hf.to({"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[precision])
    keys = MODEL_KEYS[architecture]
    heads = hf_config.num_attention_heads
    hd = hf_config.hidden_size // heads
    # ---- embeddings
    emb = torch.cat([p["word_embeddings.weight"] for p in load_partitions(input_dir, mp, 0, sequential)], dim=0)
    (hf.gpt_neox.embed_in if architecture == "neox" else hf.model.embed_tokens).load_state_dict({"weight": emb})
    layers = hf.gpt_neox.layers if architecture == "neox" else hf.model.layers
    for i in range(L):
        parts = load_partitions(input_dir, mp, i + 2, sequential)
        sd = {}
        for k, hk in keys["ROW_PARALLEL_LINEAR_KEYS"].items():
            sd[hk] = torch.cat([p[k] for p in parts], dim=1)
        for k, hk in keys["NORM_KEYS"].items():
            if k in parts[0]:
                sd[hk] = sum(p[k] for p in parts) / mp
        for k, hk in keys["ROW_PARALLEL_BIAS_KEYS"].items():
            if k in parts[0]:
                sd[hk] = sum(p[k] for p in parts)
        if architecture == "neox":
            for k, hk in keys["COLUMN_PARALLEL_LINEAR_KEYS"].items():
                if k in parts[0]:
                    sd[hk] = torch.cat([p[k] for p in parts], dim=0)
            for buf in ("attention.bias", "attention.masked_bias", "attention.rotary_emb.inv_freq"):
                if buf in layers[i].state_dict():
                    sd[buf] = layers[i].state_dict()[buf]
        else:
            kvh = hf_config.num_key_value_heads
            qs, ks, vs, ups, gates = [], [], [], [], []
            for p in parts:
                w = p["attention.query_key_value.weight"]
                if kvh == heads:          # per-head interleaved [heads/mp, 3, hd, h]
                    w = w.view(heads // mp, 3, hd, -1)
                    qs.append(w[:, 0].reshape(-1, w.shape[-1]))
                    ks.append(w[:, 1].reshape(-1, w.shape[-1]))
                    vs.append(w[:, 2].reshape(-1, w.shape[-1]))
                else:                     # contiguous [Q | K | V]
                    nq, nk = heads // mp * hd, kvh // mp * hd
                    qs.append(w[:nq]); ks.append(w[nq:nq + nk]); vs.append(w[nq + nk:])
                up, gate = torch.chunk(p["mlp.linear1.weight"], 2, dim=0)
                ups.append(up); gates.append(gate)
            sd["self_attn.q_proj.weight"] = torch.cat(qs, 0)
            sd["self_attn.k_proj.weight"] = torch.cat(ks, 0)
            sd["self_attn.v_proj.weight"] = torch.cat(vs, 0)
            sd["mlp.up_proj.weight"] = torch.cat(ups, 0)
            sd["mlp.gate_proj.weight"] = torch.cat(gates, 0)
        missing = set(layers[i].state_dict()) - set(sd)
        layers[i].load_state_dict(sd, strict=False)
    # ---- final norm + head
    parts = load_partitions(input_dir, mp, L + 3, sequential)
    fin = {hk: sum(p[k] for p in parts) / mp for k, hk in keys["FINAL_NORM_KEYS"].items() if k in parts[0]}
    (hf.gpt_neox.final_layer_norm if architecture == "neox" else hf.model.norm).load_state_dict(fin)
    if get_key(cfg, "no_weight_tying", False):
        parts = load_partitions(input_dir, mp, L + 4, sequential)
        head = torch.cat([p["final_linear.weight"] for p in parts], dim=0)
    else:
        head = emb
    (hf.embed_out if architecture == "neox" else hf.lm_head).load_state_dict({"weight": head})
    if output_dir:
        hf.save_pretrained(output_dir)
    return hf


def main(argv=None):
    ap = argparse.ArgumentParser(description="Merge a native checkpoint into a Hugging Face model directory")
    ap.add_argument("--input_dir", required=True, help="checkpoint tag directory, e.g. checkpoints/global_step143000")
    ap.add_argument("--config_file", required=True, nargs="+")
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--precision", default=None, choices=[None, "fp16", "bf16", "fp32"])
    ap.add_argument("--architecture", default="neox", choices=["neox", "llama", "mistral"])
    ap.add_argument("--no_save_tokenizer", action="store_true")
    a = ap.parse_args(argv)
    cfg = load_config(a.config_file)
    convert(a.input_dir, cfg, a.output_dir, precision=a.precision, architecture=a.architecture)
    print(f"saved Hugging Face model to {a.output_dir}")


if __name__ == "__main__":
    main()
