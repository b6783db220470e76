#!/usr/bin/env python
"""Convert a native checkpoint (sequential ``mp_rank_XX_model_states.pt`` or per-layer
``layer_XX-model_YY-model_states.pt`` files, any tensor-parallel degree) to a Hugging Face model directory.

    python -m gpt_neox_b200.tools.ckpts.convert_neox_to_hf --input_dir ckpt/global_step1000 \\
        --config_file cfg.yml --output_dir hf_out [--architecture neox|llama|mistral] [--precision auto|fp16|bf16|fp32]
        [--no_save_tokenizer] [--vocab-is-hf-tokenizer] [--pad-token-id N]

Tensor-parallel merge rules (the same ones every GPT-NeoX tool applies, ``tools/ckpts/convert_neox_to_hf.py:596-648``
of the reference): column-parallel weights and biases are concatenated along dim 0, row-parallel weights along
dim 1, norm parameters are averaged, row-parallel biases are summed.  Layout facts used:
  * fused QKV of multi-head attention is per-head interleaved ``[heads, 3, head_dim]`` -- identical to HF GPT-NeoX;
  * grouped-query QKV is contiguous ``[Q | K | V]`` per rank;
  * gated MLP ``linear1`` holds ``[up ; gate]`` halves per rank -> ``up_proj`` / ``gate_proj``;
  * checkpoints written before the MLP was renamed carry ``mlp.dense_h_to_4h`` / ``mlp.dense_4h_to_h`` (GPT-NeoX
    blocks) or ``mlp.w1`` (gate) / ``mlp.w3`` (up) / ``mlp.w2`` (down) (Llama blocks); both spellings are read;
  * a reward model (``train_impl: rm``) becomes a sequence-classification model whose ``score`` head is the
    row-parallel ``rm_linear`` merged along dim 1.
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
# spellings used by checkpoints written before the MLP modules were renamed: {old key: current key}
LEGACY_KEYS = {
    "neox": {"mlp.dense_h_to_4h.weight": "mlp.linear1.weight", "mlp.dense_h_to_4h.bias": "mlp.linear1.bias",
             "mlp.dense_4h_to_h.weight": "mlp.linear2.weight", "mlp.dense_4h_to_h.bias": "mlp.linear2.bias"},
    "llama": {"mlp.w2.weight": "mlp.linear2.weight"},       # w1 (gate) / w3 (up) are fused below
}
LEGACY_KEYS["mistral"] = LEGACY_KEYS["llama"]


def get_mlp_naming_convention(parts):
    """``"new"`` (``mlp.linear1``) or ``"legacy"`` (``mlp.dense_h_to_4h`` / ``mlp.w1``) for one layer's shards."""
    keys = set().union(*[set(p) for p in parts])
    if any("mlp.linear1.weight" in k for k in keys):
        return "new"
    if any("mlp.dense_h_to_4h.weight" in k or "mlp.w1.weight" in k for k in keys):
        return "legacy"
    raise ValueError("Unable to determine MLP naming convention in checkpoint")


def _modernise(parts, architecture):
    """Rename legacy MLP keys in place so the merge below sees one spelling."""
    for p in parts:
        for old, new in LEGACY_KEYS[architecture].items():
            if old in p:
                p[new] = p.pop(old)
        if "mlp.w1.weight" in p:                            # [up ; gate], the order linear1 keeps
            p["mlp.linear1.weight"] = torch.cat([p.pop("mlp.w3.weight"), p.pop("mlp.w1.weight")], dim=0)
    return parts


def detect_precision(cfg):
    """The 16-bit type the model was trained in (``fp16.enabled`` / ``bf16.enabled`` / ``precision``), else fp32."""
    fp16, bf16 = get_key(cfg, "fp16"), get_key(cfg, "bf16")
    prec = str(get_key(cfg, "precision", "")).lower()
    if (isinstance(bf16, dict) and bf16.get("enabled")) or prec in ("bfloat16", "bf16") or \
            (isinstance(fp16, dict) and fp16.get("type") == "bfloat16"):
        return "bf16"
    if (isinstance(fp16, dict) and fp16.get("enabled")) or prec == "fp16":
        return "fp16"
    return "fp32"


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


def create_config(cfg, architecture="neox", pad_token=0, is_rm=False, pad_token_id=-1):
    from transformers import GPTNeoXConfig, LlamaConfig, MistralConfig
    if get_key(cfg, "gpt_j_tied", False):
        raise NotImplementedError("Hugging Face GPT-NeoX has no single shared layernorm per block (gpt_j_tied); "
                                  "such a model cannot be exported")
    hf_config = _create_config(cfg, architecture, pad_token)
    if is_rm:
        hf_config.num_labels = 1
        hf_config.pad_token_id = pad_token_id
    return hf_config


def _create_config(cfg, architecture, pad_token):
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
    return LlamaConfig(**kw, attention_bias=bool(get_key(cfg, "use_bias_in_attn_linear", False)))


def convert(input_dir, cfg, output_dir=None, sequential=None, precision=None, architecture="neox", is_rm=False,
            pad_token_id=-1):
    """``precision``: ``None`` keeps fp32, ``"auto"`` takes the 16-bit type of the training config."""
    from transformers import AutoModelForCausalLM, AutoModelForSequenceClassification
    mp = get_key(cfg, "model_parallel_size", 1)
    L = get_key(cfg, "num_layers")
    if sequential is None:      # by the files: per-layer files are what a pipeline engine (pipe_parallel_size >= 1) writes
        sequential = os.path.exists(os.path.join(input_dir, "mp_rank_00_model_states.pt")) and \
            not os.path.exists(os.path.join(input_dir, "layer_00-model_00-model_states.pt"))
        print(f"checkpoint layout: {'one sequential state dict' if sequential else 'per-layer files'} per "
              "tensor-parallel rank")
    hf_config = create_config(cfg, architecture, is_rm=is_rm, pad_token_id=pad_token_id)
    hf = (AutoModelForSequenceClassification if is_rm else AutoModelForCausalLM).from_config(hf_config)
    if precision == "auto":
        precision = detect_precision(cfg)
        print(f"Auto-detected precision: saving weights in {precision}")
    if precision:
        hf = hf.to({"fp16": torch.float16, "bf16": torch.bfloat16, "fp32": torch.float32}[precision])
    keys = MODEL_KEYS[architecture]
    heads = hf_config.num_attention_heads
    hd = hf_config.hidden_size // heads
    # ---- embeddings
    emb = torch.cat([p["word_embeddings.weight"] for p in load_partitions(input_dir, mp, 0, sequential)], dim=0)
    body = hf.gpt_neox if architecture == "neox" else hf.model
    (body.embed_in if architecture == "neox" else body.embed_tokens).load_state_dict({"weight": emb})
    assert hf_config.vocab_size == emb.shape[0], \
        f"vocabulary of the config ({hf_config.vocab_size}) != embedding rows in the checkpoint ({emb.shape[0]})"
    layers = body.layers
    print(f"Detected MLP naming convention: {get_mlp_naming_convention(load_partitions(input_dir, mp, 2, sequential))}")
    for i in range(L):
        parts = _modernise(load_partitions(input_dir, mp, i + 2, sequential), architecture)
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
            if "attention.query_key_value.bias" in parts[0]:           # use_bias_in_attn_linear
                qb, kb, vb = [], [], []
                for p in parts:
                    bvec = p["attention.query_key_value.bias"]
                    if kvh == heads:
                        bvec = bvec.view(heads // mp, 3, hd)
                        qb.append(bvec[:, 0].reshape(-1)); kb.append(bvec[:, 1].reshape(-1)); vb.append(bvec[:, 2].reshape(-1))
                    else:
                        nq, nk = heads // mp * hd, kvh // mp * hd
                        qb.append(bvec[:nq]); kb.append(bvec[nq:nq + nk]); vb.append(bvec[nq + nk:])
                sd["self_attn.q_proj.bias"], sd["self_attn.k_proj.bias"], sd["self_attn.v_proj.bias"] = \
                    torch.cat(qb), torch.cat(kb), torch.cat(vb)
                if "attention.dense.bias" in parts[0]:
                    sd["self_attn.o_proj.bias"] = sum(p["attention.dense.bias"] for p in parts)
        target = layers[i].state_dict()
        for k in set(target) - set(sd):
            # a bias the Hugging Face block always has but this model was trained without: zero, not random
            assert k.endswith(".bias"), f"layer {i}: the checkpoint has nothing for {k}"
            sd[k] = torch.zeros_like(target[k])
        layers[i].load_state_dict(sd)
    # ---- final norm + head
    parts = load_partitions(input_dir, mp, L + 3, sequential)
    fin = {hk: sum(p[k] for p in parts) / mp for k, hk in keys["FINAL_NORM_KEYS"].items() if k in parts[0]}
    (body.final_layer_norm if architecture == "neox" else body.norm).load_state_dict(fin)
    if is_rm:                                     # row-parallel [1, hidden / mp] slices -> the classification head
        parts = load_partitions(input_dir, mp, L + 4, sequential)
        hf.score.load_state_dict({"weight": torch.cat([p["rm_linear.weight"] for p in parts], dim=1)})
    else:
        if get_key(cfg, "no_weight_tying", False):
            parts = load_partitions(input_dir, mp, L + 4, sequential)
            head = torch.cat([p["final_linear.weight"] for p in parts], dim=0)
        else:
            head = emb
        (hf.embed_out if architecture == "neox" else hf.lm_head).load_state_dict({"weight": head})
    if output_dir:
        hf.save_pretrained(output_dir)
    return hf


def save_tokenizer(cfg, output_dir, vocab_is_hf_tokenizer=False, pad_token_id=-1):
    """Write the tokenizer beside the model so the directory loads as one Hugging Face model.  Returns True if one
    was written (``HFTokenizer`` files and Hugging Face tokenizer folders; other tokenizer types are left out)."""
    vocab = get_key(cfg, "vocab_file")
    if vocab_is_hf_tokenizer:
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(os.path.dirname(vocab))
    elif get_key(cfg, "tokenizer_type") == "HFTokenizer":
        from transformers import PreTrainedTokenizerFast
        print(f"saving tokenizer from file {vocab}")
        print("Warning: please check that your model config and tokenizer end with the correct special tokens "
              "(EOS, BOS).")
        tok = PreTrainedTokenizerFast(tokenizer_file=vocab)
    else:
        print(f"tokenizer type {get_key(cfg, 'tokenizer_type')!r}: not saved (only HFTokenizer files and Hugging "
              "Face tokenizer folders are)")
        return False
    if pad_token_id != -1:
        tok.pad_token_id = pad_token_id
    tok.save_pretrained(output_dir)
    print("tokenizer saved!")
    return True


def main(argv=None, overwrite_values=None):
    ap = argparse.ArgumentParser(description="Merge a native checkpoint into a Hugging Face model directory")
    ap.add_argument("--input_dir", required=True, help="checkpoint tag directory, e.g. checkpoints/global_step143000")
    ap.add_argument("--config_file", required=True, nargs="+")
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--precision", default="auto", choices=["auto", "fp16", "bf16", "fp32"],
                    help="auto: the 16-bit type the config trained in, else fp32")
    ap.add_argument("--architecture", default="neox", choices=["neox", "llama", "mistral"])
    ap.add_argument("--no_save_tokenizer", action="store_true")
    ap.add_argument("--vocab-is-hf-tokenizer", action="store_true",
                    help="the vocab file sits in a Hugging Face tokenizer folder")
    ap.add_argument("--pad-token-id", type=int, default=-1, help="required for reward models")
    a = ap.parse_args(argv)
    cfg = load_config(a.config_file)
    cfg.update(overwrite_values or {})
    is_rm = get_key(cfg, "train_impl", "normal") == "rm"
    if is_rm and a.pad_token_id == -1:
        raise ValueError("RM models require a pad token id to be set.")
    convert(a.input_dir, cfg, a.output_dir, precision=a.precision, architecture=a.architecture, is_rm=is_rm,
            pad_token_id=a.pad_token_id)
    print(f"saved Hugging Face model to {a.output_dir}")
    if not a.no_save_tokenizer:
        save_tokenizer(cfg, a.output_dir, a.vocab_is_hf_tokenizer, a.pad_token_id)


if __name__ == "__main__":
    main()
