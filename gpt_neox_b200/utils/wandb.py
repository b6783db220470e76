"""Weights & Biases initialisation (``megatron/utils.py:113-187`` of the reference)."""
from __future__ import annotations

import os
import socket

from . import is_local_main, print_rank_0


def get_wandb_api_key(neox_args):
    if "WANDB_LOCAL" in os.environ:
        return "LOCAL"
    if "WANDB_API_KEY" in os.environ:
        return os.environ["WANDB_API_KEY"]
    try:
        import requests
        from urllib.parse import urlparse
        netrc = requests.utils.get_netrc_auth(urlparse(neox_args.wandb_host).geturl() if neox_args.wandb_host else "https://api.wandb.ai")
        return netrc[1] if netrc else None
    except Exception:
        return None


def init_wandb(neox_args):
    if neox_args.use_wandb is None:
        neox_args.use_wandb = False
    if not neox_args.use_wandb:
        return
    if not neox_args.wandb_init_all_ranks:
        use = is_local_main() and get_wandb_api_key(neox_args) is not None
        neox_args.use_wandb = use
    if neox_args.use_wandb:
        import wandb
        group = neox_args.wandb_group
        run_name = neox_args.wandb_run_name or f"{socket.gethostname()}-{neox_args.local_rank or 0}"
        try:
            wandb.init(project=neox_args.wandb_project, group=group, name=run_name, save_code=False, force=False,
                       entity=neox_args.wandb_team)
            wandb.config.update(neox_args.all_config)
        except Exception as exc:
            neox_args.use_wandb = False
            print_rank_0(f"Skipping wandb. Execute `wandb login` on local or main node machine to enable. ({exc})")
