"""Maximal-update parametrisation hooks (muP; Yang et al. 2022), the part the reference gets from the external
``mup`` package (``megatron/training.py:73-177``, ``megatron/mup_substitute.py``).

A *base shapes* file records the width of a small proxy model; every matrix-like parameter of the target model
gets ``mup_width_mult = fan_in / base_fan_in``.  Then: hidden weights are initialised with std / sqrt(width_mult)
(``init_functions._mup_scale``), the learning rate of matrix-like parameters is divided by the width multiplier
(Adam) through a per-group ``width_mult``, the output logits are divided by the embedding's width multiplier and
attention uses 1/d instead of 1/sqrt(d) scaling (``transformer.py``).
"""
from __future__ import annotations

import os

import yaml


def _shapes(model):
    return {name: list(p.shape) for name, p in model.named_parameters()}


def save_base_shapes(model, neox_args):
    path = neox_args.base_shapes_file or "base-shapes"
    rank = getattr(neox_args, "rank", 0) or 0
    fname = f"{path}.{rank}"
    with open(fname, "w") as fh:
        yaml.safe_dump(_shapes(model), fh)
    return fname


def apply_mup(model, neox_args):
    if neox_args.save_base_shapes:
        save_base_shapes(model, neox_args)
        return
    path = f"{neox_args.base_shapes_file}.{getattr(neox_args, 'rank', 0) or 0}" if neox_args.base_shapes_file else None
    base = {}
    if path and os.path.exists(path):
        with open(path) as fh:
            base = yaml.safe_load(fh) or {}
    for name, p in model.named_parameters():
        mult = 1.0
        shp = base.get(name)
        if shp is not None and p.dim() >= 2 and len(shp) == p.dim() and shp[-1] > 0:
            mult = p.shape[-1] / shp[-1]
        elif p.dim() >= 2 and neox_args.mup_width_scale:
            mult = float(neox_args.mup_width_scale)
        p.mup_width_mult = mult
    for m in model.modules():
        if hasattr(m, "width_mult_val") and hasattr(m, "weight"):
            m.width_mult_val = getattr(m.weight, "mup_width_mult", 1.0)


def get_coord_data(neox_args, timers, lr_scheduler, models, dataloader, optcls=None, nsteps=3, nseeds=1):
    """Coordinate check: mean absolute activation of every layer output over the first training steps for
    models of several widths; under muP these curves are flat in width.  ``models`` maps width -> constructor."""
    import pandas as pd
    import torch
    rows = []
    for width, make in models.items():
        for seed in range(nseeds):
            torch.manual_seed(seed)
            engine = make()
            hooks, records = [], {}
            for name, mod in engine.module.named_modules():
                if name:
                    hooks.append(mod.register_forward_hook(
                        lambda m, i, o, name=name: records.__setitem__(
                            name, (o[0] if isinstance(o, (tuple, list)) else o).detach().abs().mean().item()
                            if torch.is_tensor(o[0] if isinstance(o, (tuple, list)) else o) else None)))
            from .training import train_step
            for step in range(nsteps):
                records.clear()
                train_step(neox_args, timers, dataloader, engine, engine.optimizer, lr_scheduler)
                for name, val in records.items():
                    if val is not None:
                        rows.append({"width": width, "module": name, "l1": val, "t": step + 1, "seed": seed})
            for h in hooks:
                h.remove()
    return pd.DataFrame(rows)
