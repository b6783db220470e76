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


def mup_coord_check(neox_args, timers, train_data_iterator, widths=None, nsteps=3, out_dir="."):
    """The ``coord_check`` run (``megatron/training.py:139-177`` of the reference): train models of several widths for
    a few steps, once with the maximal-update parametrisation and once with the standard one, record the mean
    absolute activation of every module per step, and write ``coord_check_up.<rank>.csv`` /
    ``coord_check_sp.<rank>.csv`` (plus ``.jpg`` plots when matplotlib is importable).  Flat curves over width for
    the first file and growing ones for the second are the sign of a correct muP implementation.  Returns the two
    data frames."""
    import copy

    from .training import setup_model_and_optimizer
    base_hidden = neox_args.hidden_size
    heads = neox_args.num_attention_heads
    widths = widths or [base_hidden * (2 ** k) for k in range(3)]
    rank = getattr(neox_args, "rank", 0) or 0
    frames = {}
    keep = {k: getattr(neox_args, k) for k in ("hidden_size", "use_mup", "mup_width_scale", "save_base_shapes",
                                               "intermediate_size")}
    batches = [next(train_data_iterator) for _ in range(max(1, neox_args.gradient_accumulation_steps) * nsteps)]
    for tag, use_mup in (("up", True), ("sp", False)):
        def models():
            out = {}
            for w in widths:
                def make(w=w):
                    neox_args.hidden_size = w
                    neox_args.use_mup = use_mup
                    neox_args.save_base_shapes = False
                    neox_args.mup_width_scale = w / base_hidden
                    assert w % heads == 0
                    from .parallel import fused_comm  # noqa: F401  (same imports as a normal run)
                    engine, _, sched, _ = setup_model_and_optimizer(neox_args)
                    make.sched = sched
                    return engine
                out[w] = make
            return out

        class _Replay:
            def __init__(self):
                self.i = 0

            def __iter__(self):
                return self

            def __next__(self):
                b = batches[self.i % len(batches)]
                self.i += 1
                return copy.deepcopy(b)
        df = get_coord_data(neox_args, timers, None, models(), _Replay(), nsteps=nsteps)
        frames[tag] = df
        path = os.path.join(out_dir, f"coord_check_{tag}.{rank}")
        df.to_csv(path + ".csv", index=False)
        try:
            import matplotlib
            matplotlib.use("Agg")
            import matplotlib.pyplot as plt
            fig, axes = plt.subplots(1, nsteps, figsize=(4 * nsteps, 3))
            for t, ax in enumerate(axes if nsteps > 1 else [axes]):
                for mod, g in df[df.t == t + 1].groupby("module"):
                    ax.plot(g.width, g.l1, alpha=0.4)
                ax.set_xscale("log", base=2)
                ax.set_yscale("log")
                ax.set_title(f"t={t + 1}")
            fig.savefig(path + ".jpg")
            plt.close(fig)
        except Exception:
            pass
    for k, v in keep.items():
        setattr(neox_args, k, v)
    return frames["up"], frames["sp"]
