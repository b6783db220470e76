#!/usr/bin/env python
"""Evaluate a checkpoint on lm-eval-harness tasks: ``./deepy.py eval.py <configs> --eval_tasks lambada piqa``
(``eval.py:34-75`` of the reference).  Results go to stdout, W&B / TensorBoard and a JSON file."""
import json
import os
import sys
from datetime import datetime

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(input_args=None, overwrite_values=None):
    from pprint import pprint
    from gpt_neox_b200.eval_tasks import run_eval_harness
    from gpt_neox_b200.logging import tb_wandb_log
    from gpt_neox_b200.training import forward_step
    from gpt_neox_b200.utils import is_rank_0 as _r0, setup_for_inference_or_eval
    from gpt_neox_b200.utils.wandb import init_wandb
    model, neox_args = setup_for_inference_or_eval(use_cache=False, input_args=input_args,
                                                   overwrite_values=overwrite_values)
    results = run_eval_harness(model, forward_step, neox_args, eval_tasks=neox_args.eval_tasks,
                               bootstrap_iters=10000)
    if neox_args.rank == 0:
        init_wandb(neox_args=neox_args)
        for k, v in results["results"].items():
            if isinstance(v, dict):
                for k2, v2 in v.items():
                    if isinstance(v2, (int, float)):
                        tb_wandb_log(f"eval/{k}_{k2}", v2, neox_args.iteration, use_wandb=neox_args.use_wandb,
                                     comet_experiment=neox_args.comet_experiment)
        pprint(results)
        results_path = f'eval_results_{datetime.now().strftime("%m-%d-%Y-%H-%M-%S")}.json'
        if neox_args.eval_results_prefix:
            results_path = f"{neox_args.eval_results_prefix}_{results_path}"
        with open(results_path, "w") as fh:
            json.dump(results, fh, indent=4, default=str)


if __name__ == "__main__":
    main()
