"""FLOPs profiler: per-module parameters, forward multiply-accumulates and forward latency of one training step.

The reference forwards its ``flops_profiler`` block (``enabled / profile_step / module_depth / top_modules /
detailed / output_file``, ``megatron/neox_arguments/deepspeed_args.py:158``) to DeepSpeed, whose profiler patches
``torch.nn.functional`` to count operations.  Here the arithmetic that matters runs in this package's own kernels,
so the counting sits at their front-ends: ``ops.gemm.gemm`` / ``ops.fp8.gemm_fp8`` / the eager linear fallback add
``2 M N K`` and the attention entry points add ``4 b h s_q s_k d`` (halved for a causal mask) through ``ops.flop_count``.
Module forward hooks attribute the counter's growth and the elapsed device time to each module (inclusive of its
children), the way the DeepSpeed report is organised.  Recomputed forwards (activation checkpointing) are not
counted twice.
"""
from __future__ import annotations

import time

import torch

from ..ops import flop_count


class FlopsProfiler:
    def __init__(self, model, enabled=False, profile_step=1, module_depth=-1, top_modules=1, detailed=True,
                 output_file=None):
        self.model, self.enabled = model, bool(enabled)
        self.profile_step, self.module_depth, self.top_modules = int(profile_step), int(module_depth), int(top_modules)
        self.detailed, self.output_file = bool(detailed), output_file
        self.flops, self._on = 0.0, False
        self._hooks, self._stack, self.stats = [], [], {}
        self._t_start = self._t_fwd_end = self._t_end = None

    @property
    def counting(self):
        # only arithmetic issued inside a (first, not recomputed) module forward counts: backward GEMMs and
        # recomputation go through the same front-ends
        return self._on and bool(self._stack) and self._stack[-1] is not None

    @classmethod
    def from_config(cls, model, block):
        block = dict(block or {})
        return cls(model, **{k: block[k] for k in ("enabled", "profile_step", "module_depth", "top_modules", "detailed",
                                                   "output_file") if k in block})

    # ------------------------------------------------------------------ hooks
    def _now(self):
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
            return e
        return time.perf_counter()

    @staticmethod
    def _elapsed_ms(a, b):
        if isinstance(a, float):
            return (b - a) * 1e3
        return a.elapsed_time(b)

    def _pre(self, name):
        def hook(module, args):
            from ..parallel.rng import in_recompute
            if in_recompute():
                self._stack.append(None)
                return
            self._stack.append((name, self.flops, self._now()))
        return hook

    def _post(self, name):
        def hook(module, args, output):
            top = self._stack.pop() if self._stack else None
            if top is None:
                return
            _, f0, t0 = top
            st = self.stats.setdefault(name, {"flops": 0.0, "spans": [], "calls": 0})
            st["flops"] += self.flops - f0
            st["spans"].append((t0, self._now()))
            st["calls"] += 1
        return hook

    def start_profile(self):
        """Install the hooks and start counting (call right before the profiled step)."""
        self.flops, self.stats, self._stack = 0.0, {}, []
        for name, mod in self.model.named_modules():
            self._hooks.append(mod.register_forward_pre_hook(self._pre(name)))
            self._hooks.append(mod.register_forward_hook(self._post(name)))
        flop_count.ACTIVE[0], self._on = self, True
        self._t_start = self._now()

    def stop_profile(self):
        self._t_end = self._now()
        self._on = False
        if flop_count.ACTIVE[0] is self:
            flop_count.ACTIVE[0] = None
        for h in self._hooks:
            h.remove()
        self._hooks = []
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        for st in self.stats.values():
            st["ms"] = sum(self._elapsed_ms(a, b) for a, b in st.pop("spans"))
        if "" not in self.stats:
            # a pipeline stage runs its layers one by one and never calls the container's forward
            top = [st for name, st in self.stats.items() if "." not in name]
            self.stats[""] = {"flops": self.flops, "ms": sum(st["ms"] for st in top), "calls": 1}

    # ------------------------------------------------------------------ report
    def total_flops(self):
        return self.stats.get("", {}).get("flops", self.flops)

    def total_params(self):
        return sum(p.numel() for p in self.model.parameters())

    def report(self, batch_size=None):
        step_ms = self._elapsed_ms(self._t_start, self._t_end)
        fwd = self.stats.get("", {"flops": self.flops, "ms": 0.0, "calls": 0})
        lines = ["-------------------------- Flops Profiler --------------------------",
                 f"Profile on step {self.profile_step} (this rank's shard of the model):",
                 f"params per GPU:                     {_num(self.total_params())}",
                 f"fwd MACs per GPU:                   {_num(fwd['flops'] / 2)}MACs",
                 f"fwd flops per GPU:                  {_num(fwd['flops'])}",
                 f"fwd latency:                        {fwd['ms']:.2f} ms",
                 f"fwd FLOPS per GPU:                  {_num(fwd['flops'] / max(fwd['ms'], 1e-9) * 1e3)}FLOPS",
                 f"fwd+bwd flops per GPU (bwd = 2 fwd): {_num(3 * fwd['flops'])}",
                 f"step latency (fwd+bwd+optimizer):   {step_ms:.2f} ms",
                 f"step FLOPS per GPU:                 {_num(3 * fwd['flops'] / max(step_ms, 1e-9) * 1e3)}FLOPS"]
        if batch_size:
            lines.append(f"samples/second:                     {batch_size / max(step_ms, 1e-9) * 1e3:.2f}")
        by_depth = {}
        for name, st in self.stats.items():
            depth = 0 if name == "" else name.count(".") + 1
            by_depth.setdefault(depth, []).append((name or type(self.model).__name__, st))
        max_depth = max(by_depth) if by_depth else 0
        depth_limit = max_depth if self.module_depth < 0 else min(self.module_depth, max_depth)
        lines.append("")
        lines.append(f"Aggregated profile per depth (top {self.top_modules} by forward latency):")
        for depth in range(depth_limit + 1):
            mods = sorted(by_depth.get(depth, []), key=lambda kv: -kv[1]["ms"])[: max(self.top_modules, 1)]
            lines.append(f"depth {depth}:")
            for name, st in mods:
                lines.append(f"    {name}: {_num(st['flops'] / 2)}MACs, {st['ms']:.3f} ms, {st['calls']} call(s)")
        if self.detailed:
            lines.append("")
            lines.append("Detailed profile per module (params, fwd MACs, fwd latency, share of fwd latency):")
            params = {n: sum(p.numel() for p in m.parameters()) for n, m in self.model.named_modules()}
            for name, mod in self.model.named_modules():
                depth = 0 if name == "" else name.count(".") + 1
                if depth > depth_limit or name not in self.stats:
                    continue
                st = self.stats[name]
                share = 100.0 * st["ms"] / max(fwd["ms"], 1e-9)
                lines.append(f"{'  ' * depth}{name or type(mod).__name__} ({type(mod).__name__}): "
                             f"{_num(params[name])}, {_num(st['flops'] / 2)}MACs, {st['ms']:.3f} ms, {share:.1f}%")
        lines.append("---------------------------------------------------------------------")
        text = "\n".join(lines)
        if self.output_file:
            with open(self.output_file, "w") as f:
                f.write(text + "\n")
        return text


def _num(x):
    x = float(x)
    for unit, div in (("T", 1e12), ("G", 1e9), ("M", 1e6), ("K", 1e3)):
        if abs(x) >= div:
            return f"{x / div:.2f} {unit}"
    return f"{x:.0f} "
