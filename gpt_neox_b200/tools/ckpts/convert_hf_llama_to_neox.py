"""Hugging Face Llama / Mistral checkpoint -> tensor-parallel NeoX sequential checkpoint.

    python -m gpt_neox_b200.tools.ckpts.convert_hf_llama_to_neox --model meta-llama/Llama-2-7b-hf \
        --output_dir ckpts/llama2-7b --tp 4

Sharding rules (same as ``tools/ckpts/convert_hf_llama_to_neox.py`` of the reference): embeddings and LM head split
along the vocabulary, q / k / v fused per rank (interleaved per head for MHA, ``[Q | K | V]`` blocks for grouped-query
attention), ``o_proj`` and ``down_proj`` split along their input dimension, ``up_proj`` and ``gate_proj`` concatenated
as ``[up; gate]`` per rank, RMSNorm scales replicated.  The work is done by ``convert_hf_to_sequential.convert``; this
entry point only fixes the architecture and also writes the matching tokenizer files when asked to.
"""
import argparse

from .convert_hf_to_sequential import convert, save


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", required=True, help="HF hub id or local directory of a Llama-family model")
    ap.add_argument("--output_dir", required=True)
    ap.add_argument("--tp", type=int, default=1, help="tensor-parallel degree of the output checkpoint")
    ap.add_argument("--save_tokenizer", action="store_true", help="also save the tokenizer beside the checkpoint")
    a = ap.parse_args(argv)
    import torch
    from transformers import AutoModelForCausalLM, AutoTokenizer
    hf = AutoModelForCausalLM.from_pretrained(a.model, torch_dtype=torch.bfloat16)
    save(convert(hf, a.tp, "llama"), a.output_dir)
    if a.save_tokenizer:
        AutoTokenizer.from_pretrained(a.model).save_pretrained(a.output_dir)
    print(f"wrote {a.tp} model-parallel shard(s) to {a.output_dir}/global_step0")


if __name__ == "__main__":
    main()
