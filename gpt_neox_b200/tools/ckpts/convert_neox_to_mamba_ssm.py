"""NeoX Mamba checkpoint -> the ``state-spaces/mamba`` (``mamba_ssm`` ``MambaLMHeadModel``) state-dict layout.

    python -m gpt_neox_b200.tools.ckpts.convert_neox_to_mamba_ssm --input_dir ckpts/mamba/global_step1000 \
        --config_file configs/mamba/mamba-130M.yml --output_dir out/mamba-130m

Tensor-parallel shards are merged first: ``in_proj`` is column-parallel with the ``x`` and ``z`` halves interleaved per
rank, so the halves are concatenated separately; ``conv1d``, ``dt_proj``, ``A_log`` and ``D`` are sharded along the inner
dimension; ``x_proj`` and ``out_proj`` are row-parallel (concatenate along dim 1); norms are averaged.  The result is
written as ``pytorch_model.bin`` + ``config.json`` (``d_model``, ``n_layer``, ``vocab_size``, ``ssm_cfg``), which
``MambaLMHeadModel.from_pretrained`` of the reference implementation loads; that package is not needed to convert
(the reference tool, ``tools/ckpts/convert_neox_to_mamba_ssm.py``, instantiates the model to copy into it).
"""
import argparse
import json
import os

import torch

from .convert_neox_to_hf import get_key, load_config, load_partitions


def convert(input_dir, cfg, sequential=None):
    mp = get_key(cfg, "model_parallel_size", 1)
    L = get_key(cfg, "num_layers")
    if sequential is None:
        sequential = not os.path.exists(os.path.join(input_dir, "layer_00-model_00-model_states.pt"))
    out = {}
    emb = torch.cat([p["word_embeddings.weight"] for p in load_partitions(input_dir, mp, 0, sequential)], dim=0)
    out["backbone.embedding.weight"] = emb
    for i in range(L):
        parts = load_partitions(input_dir, mp, i + 2, sequential)
        pre = f"backbone.layers.{i}."
        xs, zs = zip(*[torch.chunk(p["mixer.in_proj.weight"], 2, dim=0) for p in parts])
        out[pre + "mixer.in_proj.weight"] = torch.cat(list(xs) + list(zs), dim=0)
        for k in ("mixer.conv1d.weight", "mixer.conv1d.bias", "mixer.dt_proj.weight", "mixer.dt_proj.bias",
                  "mixer.A_log", "mixer.D"):
            if k in parts[0]:
                out[pre + k] = torch.cat([p[k] for p in parts], dim=0)
        for k in ("mixer.x_proj.weight", "mixer.out_proj.weight"):
            out[pre + k] = torch.cat([p[k] for p in parts], dim=1)
        for k, nk in (("norm.scale", "norm.weight"), ("norm.weight", "norm.weight"), ("norm.bias", "norm.bias")):
            if k in parts[0]:
                out[pre + nk] = sum(p[k] for p in parts) / mp
    parts = load_partitions(input_dir, mp, L + 3, sequential)
    for k, nk in (("norm.scale", "backbone.norm_f.weight"), ("norm.weight", "backbone.norm_f.weight"),
                  ("norm.bias", "backbone.norm_f.bias")):
        if k in parts[0]:
            out[nk] = sum(p[k] for p in parts) / mp
    if get_key(cfg, "no_weight_tying", False):
        parts = load_partitions(input_dir, mp, L + 4, sequential)
        out["lm_head.weight"] = torch.cat([p["final_linear.weight"] for p in parts], dim=0)
    else:
        out["lm_head.weight"] = emb
    config = {"d_model": get_key(cfg, "hidden_size"), "n_layer": L, "vocab_size": emb.shape[0],
              "ssm_cfg": {}, "rms_norm": get_key(cfg, "norm", "layernorm") == "rmsnorm",
              "residual_in_fp32": False, "fused_add_norm": True, "pad_vocab_size_multiple": 1,
              "tie_embeddings": not get_key(cfg, "no_weight_tying", False)}
    return out, config


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input_dir", required=True, help="checkpoint step directory (global_stepN)")
    ap.add_argument("--config_file", required=True, help="the model's YAML config")
    ap.add_argument("--output_dir", required=True)
    a = ap.parse_args(argv)
    sd, config = convert(a.input_dir, load_config(a.config_file))
    os.makedirs(a.output_dir, exist_ok=True)
    torch.save(sd, os.path.join(a.output_dir, "pytorch_model.bin"))
    with open(os.path.join(a.output_dir, "config.json"), "w") as fh:
        json.dump(config, fh, indent=2)
    print(f"wrote {len(sd)} tensors to {a.output_dir}")


if __name__ == "__main__":
    main()
