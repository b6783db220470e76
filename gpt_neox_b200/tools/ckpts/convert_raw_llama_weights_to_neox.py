"""Meta's original Llama release (``consolidated.XX.pth`` + ``params.json``) -> NeoX checkpoint.

    python -m gpt_neox_b200.tools.ckpts.convert_raw_llama_weights_to_neox --input_dir llama/7B \
        --output_dir ckpts/llama-7b --num_output_shards 2 [--pipeline_parallel]

The raw shards are tensor-parallel pieces: ``wq/wk/wv/w1/w3`` and the output head are split along dim 0,
``wo/w2`` and the token embedding along dim 1.  They are merged to full matrices first, then re-sharded for the
requested tensor-parallel degree with the NeoX layout:

* q and k use the interleaved rotary convention (pairs ``(2i, 2i+1)``); NeoX rotates halves, so each head's rows are
  permuted ``[0, 2, 4, ..., 1, 3, 5, ...]`` (``permute_rotary`` in the reference tool of the same name);
* fused QKV per rank: per-head ``[q; k; v]`` for MHA, ``[Q | K | V]`` blocks for GQA;
* ``mlp.linear1 = [w3; w1]`` (up, then gate) and ``mlp.linear2 = w2``.

Output: ``mp_rank_XX_model_states.pt`` (sequential layout) or, with ``--pipeline_parallel``,
``layer_XX-model_YY-model_states.pt`` files, plus ``latest``.
"""
import argparse
import glob
import json
import os

import torch


def _merge(shards, key, dim):
    parts = [s[key] for s in shards]
    return parts[0] if len(parts) == 1 or dim is None else torch.cat(parts, dim=dim)


def permute_rotary(w, n_heads, head_dim):
    """Interleaved-pair rotary rows -> rotate-half rows, per head."""
    h = w.shape[-1]
    return w.view(n_heads, head_dim // 2, 2, h).transpose(1, 2).reshape(n_heads * head_dim, h)


def convert(input_dir, tp):
    params = json.load(open(os.path.join(input_dir, "params.json")))
    files = sorted(glob.glob(os.path.join(input_dir, "consolidated.*.pth")))
    assert files, f"no consolidated.*.pth under {input_dir}"
    shards = [torch.load(f, map_location="cpu") for f in files]
    L, heads, dim = params["n_layers"], params["n_heads"], params["dim"]
    kvh = params.get("n_kv_heads", heads) or heads
    hd = dim // heads
    out = [dict() for _ in range(tp)]

    def put(idx, name, tensors):
        for r in range(tp):
            out[r][f"sequential.{idx}.{name}"] = tensors[r].clone().contiguous()

    split = lambda t, d: list(torch.chunk(t, tp, dim=d))
    rep = lambda t: [t] * tp
    put(0, "word_embeddings.weight", split(_merge(shards, "tok_embeddings.weight", 1), 0))
    for i in range(L):
        p = f"layers.{i}."
        q = permute_rotary(_merge(shards, p + "attention.wq.weight", 0), heads, hd)
        k = permute_rotary(_merge(shards, p + "attention.wk.weight", 0), kvh, hd)
        v = _merge(shards, p + "attention.wv.weight", 0)
        fused = []
        for r in range(tp):
            if kvh == heads:
                n = heads // tp
                sl = slice(r * n, (r + 1) * n)
                fused.append(torch.stack([q.view(heads, hd, -1)[sl], k.view(heads, hd, -1)[sl],
                                          v.view(heads, hd, -1)[sl]], dim=1).reshape(n * 3 * hd, -1))
            else:
                nq, nk = heads // tp * hd, kvh // tp * hd
                fused.append(torch.cat([q[r * nq:(r + 1) * nq], k[r * nk:(r + 1) * nk], v[r * nk:(r + 1) * nk]], 0))
        put(i + 2, "attention.query_key_value.weight", fused)
        put(i + 2, "attention.dense.weight", split(_merge(shards, p + "attention.wo.weight", 1), 1))
        ups = split(_merge(shards, p + "feed_forward.w3.weight", 0), 0)
        gates = split(_merge(shards, p + "feed_forward.w1.weight", 0), 0)
        put(i + 2, "mlp.linear1.weight", [torch.cat([u, g], 0) for u, g in zip(ups, gates)])
        put(i + 2, "mlp.linear2.weight", split(_merge(shards, p + "feed_forward.w2.weight", 1), 1))
        put(i + 2, "input_layernorm.scale", rep(shards[0][p + "attention_norm.weight"]))
        put(i + 2, "post_attention_layernorm.scale", rep(shards[0][p + "ffn_norm.weight"]))
    put(L + 3, "norm.scale", rep(shards[0]["norm.weight"]))
    put(L + 4, "final_linear.weight", split(_merge(shards, "output.weight", 0), 0))
    return out, params


def save(shards, output_dir, pipeline_parallel=False, tag="global_step0"):
    d = os.path.join(output_dir, tag)
    os.makedirs(d, exist_ok=True)
    if not pipeline_parallel:
        from .convert_hf_to_sequential import save as save_seq
        return save_seq(shards, output_dir, tag)
    for r, sd in enumerate(shards):
        by_layer = {}
        for key, t in sd.items():
            _, idx, name = key.split(".", 2)
            by_layer.setdefault(int(idx), {})[name] = t
        for idx, layer_sd in by_layer.items():
            torch.save(layer_sd, os.path.join(d, f"layer_{idx:02d}-model_{r:02d}-model_states.pt"))
        torch.save({"dp_world_size": 1, "mp_world_size": len(shards), "optimizer": None, "global_steps": 0,
                    "skipped_steps": 0, "iteration": 0}, os.path.join(d, f"mp_rank_{r:02d}_model_states.pt"))
    with open(os.path.join(output_dir, "latest"), "w") as fh:
        fh.write(tag)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input_dir", required=True, help="directory with params.json and consolidated.XX.pth")
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--num_output_shards", type=int, default=1, help="tensor-parallel degree of the output")
    ap.add_argument("--pipeline_parallel", action="store_true", help="write one file per layer (pipeline layout)")
    a = ap.parse_args(argv)
    shards, params = convert(a.input_dir, a.num_output_shards)
    save(shards, a.output_dir, a.pipeline_parallel)
    print(f"converted {params['n_layers']} layers, hidden {params['dim']} -> {a.output_dir}")


if __name__ == "__main__":
    main()
