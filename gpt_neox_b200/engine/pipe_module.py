"""Layer specifications and the stage-partitioned module container.

The reference builds its model as a flat list of ``LayerSpec`` / ``TiedLayerSpec`` / plain callables
and hands it to DeepSpeed's ``PipelineModule`` (``megatron/model/gpt2_model.py:96-144``), which
instantiates only the layers owned by the local pipeline stage.  This file provides that container:

* ``partition_method``: ``uniform`` (equal layer counts), ``parameters`` (balance parameter counts)
  or ``type:<regex>`` (balance the number of layers whose class name matches, the default
  ``type:transformer|mlp``);
* layer ``idx`` = position in the spec list; it names checkpoint files
  (``layer_{idx:02d}-model_{tp:02d}-model_states.pt``) and sequential state-dict keys
  (``sequential.{idx}.<param>``);
* tied layers (``TiedLayerSpec`` with the same key) share one module per stage; stages that hold a
  copy all-reduce its gradient over the group of owning stages each step;
* activation checkpointing every ``activation_checkpoint_interval`` layers with RNG replay.
"""
from __future__ import annotations

import contextlib
import re

import torch
import torch.distributed as dist
import torch.nn as nn

from ..parallel import mpu
from ..parallel.rng import set_block_tail
from ..parallel.rng import checkpoint as ckpt_fn


class LayerSpec:
    """Deferred construction of a layer: ``LayerSpec(cls, *args, **kwargs).build()``."""

    def __init__(self, typename, *module_args, **module_kwargs):
        if not issubclass(typename, nn.Module):
            raise RuntimeError("LayerSpec only supports torch.nn.Module types.")
        self.typename, self.module_args, self.module_kwargs = typename, module_args, module_kwargs

    # set by ``built_through``: called on every freshly built layer (e.g. to park it in host memory)
    _post_build = None

    def build(self):
        module = self.typename(*self.module_args, **self.module_kwargs)
        hook = LayerSpec._post_build
        if hook is not None and not any(p.is_meta for p in module.parameters()):
            module = hook(module) or module
        return module

    def __repr__(self):
        return f"LayerSpec({self.typename.__name__})"


class TiedLayerSpec(LayerSpec):
    def __init__(self, key, typename, *module_args, forward_fn=None, tied_weight_attr="weight", **module_kwargs):
        super().__init__(typename, *module_args, **module_kwargs)
        self.key, self.forward_fn, self.tied_weight_attr = key, forward_fn, tied_weight_attr


@contextlib.contextmanager
def built_through(hook):
    """Inside the block every layer built from a ``LayerSpec`` is passed through ``hook(module)`` as soon as it
    exists, before the next one is built."""
    prev = LayerSpec._post_build
    LayerSpec._post_build = hook
    try:
        yield
    finally:
        LayerSpec._post_build = prev


def partition_uniform(num_items, num_parts):
    parts = [0] * (num_parts + 1)
    if num_items <= num_parts:
        for p in range(num_parts + 1):
            parts[p] = min(p, num_items)
        return parts
    chunk, rem = divmod(num_items, num_parts)
    for p in range(num_parts):
        parts[p + 1] = parts[p] + chunk + (1 if p < rem else 0)
    return parts


def partition_balanced(weights, num_parts):
    """Contiguous partition minimising the heaviest part (binary search over the bottleneck)."""
    n = len(weights)
    if n <= num_parts:
        return partition_uniform(n, num_parts)

    def parts_for(limit):
        bounds, acc, used = [0], 0, 1
        for i, w in enumerate(weights):
            if w > limit:
                return None
            if acc + w > limit:
                bounds.append(i)
                acc, used = w, used + 1
                if used > num_parts:
                    return None
            else:
                acc += w
        while len(bounds) < num_parts:
            bounds.append(n)
        bounds.append(n)
        return bounds

    lo, hi = max(weights), sum(weights)
    best = parts_for(hi)
    while lo < hi:
        mid = (lo + hi) // 2
        cand = parts_for(mid)
        if cand is not None:
            best, hi = cand, mid
        else:
            lo = mid + 1
    return best


class PipelineModule(nn.Module):
    def __init__(self, layers, num_stages=None, topology=None, loss_fn=None, seed_layers=False, base_seed=1234,
                 partition_method="parameters", activation_checkpoint_interval=0, activation_checkpoint_func=ckpt_fn,
                 checkpointable_layers=None):
        super().__init__()
        self._layer_specs = list(layers)
        self.loss_fn = loss_fn
        self.activation_checkpoint_interval = activation_checkpoint_interval
        self.activation_checkpoint_func = activation_checkpoint_func
        self.checkpointable_layers = checkpointable_layers
        self.num_stages = num_stages if num_stages is not None else max(1, mpu.get_pipe_parallel_world_size())
        self.stage_id = mpu.get_pipe_parallel_rank() if self.num_stages > 1 else 0
        self._topo = topology
        self.forward_funcs, self.fwd_map = [], {}
        self.tied_modules = nn.ModuleDict()
        self.tied_weight_attrs = {}
        self.tied_specs = {}
        self._partition_layers(partition_method)
        self._build()
        self.tied_comms = self._index_tied_modules()

    # ------------------------------------------------------------------ partitioning
    def _count_layer_params(self):
        counts = []
        for spec in self._layer_specs:
            if isinstance(spec, LayerSpec):
                # build on the meta device to count without allocating
                try:
                    with torch.device("meta"):
                        m = spec.build()
                    counts.append(sum(p.numel() for p in m.parameters()))
                except Exception:
                    counts.append(1)
            elif isinstance(spec, nn.Module):
                counts.append(sum(p.numel() for p in spec.parameters()))
            else:
                counts.append(0)
        return counts

    def _find_layer_type(self, layername):
        rx = re.compile(layername, re.IGNORECASE)
        idxs = []
        for i, spec in enumerate(self._layer_specs):
            if isinstance(spec, LayerSpec):
                name = spec.typename.__name__
            elif isinstance(spec, nn.Module):
                name = spec.__class__.__name__
            else:
                name = getattr(spec, "__name__", "")
            if rx.search(name):
                idxs.append(i)
        return idxs

    def _partition_layers(self, method="uniform"):
        n = len(self._layer_specs)
        method = method.lower()
        if method == "uniform":
            self.parts = partition_uniform(n, self.num_stages)
        elif method == "parameters":
            self.parts = partition_balanced(self._count_layer_params(), self.num_stages)
        elif method.startswith("type:"):
            weights = [0] * n
            for i in self._find_layer_type(method.split(":", 1)[1]):
                weights[i] = 1
            self.parts = partition_balanced(weights, self.num_stages)
        else:
            raise NotImplementedError(f"Partitioning method {method} not implemented.")
        self.parts[0], self.parts[-1] = 0, n
        self._local_start, self._local_stop = self.parts[self.stage_id], self.parts[self.stage_id + 1]

    def stage_owner(self, layer_idx):
        for s in range(self.num_stages):
            if self.parts[s] <= layer_idx < self.parts[s + 1]:
                return s
        raise RuntimeError(f"Layer {layer_idx} not owned? parts={self.parts}")

    # ------------------------------------------------------------------ construction
    def _build(self):
        for local_idx, spec in enumerate(self._layer_specs[self._local_start:self._local_stop]):
            idx = local_idx + self._local_start
            if isinstance(spec, nn.Module):
                self.forward_funcs.append(spec)
                self.fwd_map[str(idx)] = len(self.forward_funcs) - 1
                self.add_module(str(idx), spec)
            elif isinstance(spec, TiedLayerSpec):
                if spec.key not in self.tied_modules:
                    self.tied_modules[spec.key] = spec.build()
                    self.tied_weight_attrs[spec.key] = spec.tied_weight_attr
                self.tied_specs.setdefault(spec.key, []).append(idx)
                mod = self.tied_modules[spec.key]
                if spec.forward_fn is None:
                    self.forward_funcs.append(mod)
                else:
                    fn = spec.forward_fn
                    self.forward_funcs.append(lambda x, _m=mod, _f=fn: _f(_m, x))
            elif isinstance(spec, LayerSpec):
                mod = spec.build()
                self.forward_funcs.append(mod)
                self.fwd_map[str(idx)] = len(self.forward_funcs) - 1
                self.add_module(str(idx), mod)
            else:
                self.forward_funcs.append(spec)

    def _index_tied_modules(self):
        """For each tied key: the pipeline stages holding a copy and (if >1) a process group over them."""
        comms = {}
        keys = sorted({s.key for s in self._layer_specs if isinstance(s, TiedLayerSpec)})
        for key in keys:
            stages = sorted({self.stage_owner(i) for i, s in enumerate(self._layer_specs)
                             if isinstance(s, TiedLayerSpec) and s.key == key})
            group, ranks_mine = None, None
            if len(stages) > 1 and dist.is_available() and dist.is_initialized():
                topo = mpu.get_topology()
                for d in range(topo.dp):
                    for m in range(topo.mp):
                        ranks = [topo.rank(s, d, m) for s in stages]
                        g = dist.new_group(ranks)
                        if dist.get_rank() in ranks:
                            group, ranks_mine = g, ranks
            comms[key] = {"stages": stages, "group": group, "ranks": ranks_mine,
                          "weight_attr": self.tied_weight_attrs.get(key)}
            uses = sum(1 for s in self._layer_specs if isinstance(s, TiedLayerSpec) and s.key == key)
            if uses > 1 and key in self.tied_modules:
                # several uses (possibly on other stages) contribute to this gradient: an optimizer that reduces
                # gradients early over the data-parallel group must leave it until the whole backward and the
                # tied all-reduce have finished
                self.tied_weight(key).late_grad_sync = True
        return comms

    def tied_weight(self, key):
        mod = self.tied_modules[key]
        obj = mod
        for part in self.tied_weight_attrs[key].split("."):
            obj = getattr(obj, part)
        return obj

    def allreduce_tied_weight_gradients(self):
        for key, comm in self.tied_comms.items():
            if comm["group"] is None or key not in self.tied_modules:
                continue
            w = self.tied_weight(key)
            g = getattr(w, "main_grad", None)
            if g is None:
                g = w.grad
            if g is not None:
                dist.all_reduce(g, group=comm["group"])

    def sync_tied_weights(self):
        """Broadcast each tied weight from its first owning stage (called once after init)."""
        for key, comm in self.tied_comms.items():
            if comm["group"] is None or key not in self.tied_modules:
                continue
            dist.broadcast(self.tied_weight(key).data, src=min(comm["ranks"]), group=comm["group"])

    # ------------------------------------------------------------------ execution
    def _is_checkpointable(self, funcs):
        if self.checkpointable_layers is not None:
            return all(f.__class__.__name__ in self.checkpointable_layers for f in funcs)
        if all("ParallelTransformerLayerPipe" in f.__class__.__name__ for f in funcs):
            return True
        return any(isinstance(f, nn.Module) and any(True for _ in f.parameters()) for f in funcs)

    def exec_range(self, start, end):
        def run(*inputs):
            x = inputs[0] if len(inputs) == 1 else inputs
            block = self.forward_funcs[start:end]
            for i, f in enumerate(block):
                set_block_tail(i == len(block) - 1)
                x = f(x)
            return x
        return run

    def forward(self, forward_input):
        n = len(self.forward_funcs)
        interval = self.activation_checkpoint_interval
        if interval == 0 or not torch.is_grad_enabled():
            return self.exec_range(0, n)(forward_input)
        x = forward_input
        for start in range(0, n, interval):
            end = min(start + interval, n)
            funcs = self.forward_funcs[start:end]
            if not isinstance(x, tuple):
                x = (x,)
            if self._is_checkpointable(funcs):
                x = self.activation_checkpoint_func(self.exec_range(start, end), *x)
            else:
                x = self.exec_range(start, end)(*x)
        return x

    # ------------------------------------------------------------------ checkpoint helpers
    def local_layer_indices(self):
        return list(range(self._local_start, self._local_stop))

    def layer_module(self, idx):
        """The nn.Module at global spec index ``idx`` on this stage (tied layers included), or None."""
        if str(idx) in self._modules:
            return self._modules[str(idx)]
        spec = self._layer_specs[idx]
        if isinstance(spec, TiedLayerSpec) and self._local_start <= idx < self._local_stop:
            return self.tied_modules[spec.key]
        return None

    def num_pipeline_layers(self):
        return len(self._layer_specs)
