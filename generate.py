#!/usr/bin/env python
"""Text generation: ``./deepy.py generate.py <configs> [-i prompts.txt -o samples.txt]``.
``text_gen_type``: unconditional | input-file | interactive | precompute (``generate.py:30-92`` of the reference)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(input_args=None, overwrite_values=None):
    from gpt_neox_b200.text_generation import (generate_samples_from_prompt, generate_samples_input_from_file,
                                               generate_samples_interactive, generate_samples_unconditional,
                                               precompute_logits)
    from gpt_neox_b200.utils import print_rank_0, setup_for_inference_or_eval
    model, neox_args = setup_for_inference_or_eval(use_cache=True, input_args=input_args,
                                                   overwrite_values=overwrite_values)
    if neox_args.recompute:
        model.module.inference_mode(use_cache=False)
    print_rank_0(f"Generating samples in {neox_args.text_gen_type} mode")
    kw = dict(maximum_tokens=neox_args.maximum_tokens, recompute=neox_args.recompute,
              temperature=neox_args.temperature, top_k=neox_args.top_k, top_p=neox_args.top_p)
    if neox_args.text_gen_type == "unconditional":
        print_rank_0(f"Generating samples unconditionally and saving results to {neox_args.sample_output_file}")
        generate_samples_unconditional(neox_args=neox_args, model=model, number_of_samples=neox_args.num_samples,
                                       output_file=neox_args.sample_output_file, **kw)
    elif neox_args.text_gen_type == "input-file":
        print_rank_0(f"Generating samples from input file {neox_args.sample_input_file}")
        assert neox_args.sample_input_file is not None
        generate_samples_input_from_file(neox_args=neox_args, model=model, input_file=neox_args.sample_input_file,
                                         output_file=neox_args.sample_output_file, **kw)
    elif neox_args.text_gen_type == "interactive":
        generate_samples_interactive(neox_args=neox_args, model=model, **kw)
    elif neox_args.text_gen_type == "precompute":
        precompute_logits(neox_args=neox_args, model=model)
    else:
        raise ValueError(f"`text_gen_type` either not specified or not recognised: {neox_args.text_gen_type}")


if __name__ == "__main__":
    main()
