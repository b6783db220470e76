"""Layer-spec list -> the layers owned by this pipeline stage (what the reference's GPT2ModelPipe extends)."""
import collections
import re

import torch
import torch.distributed as dist

from ..activation_checkpointing import checkpointing


class LayerSpec:
    def __init__(self, typename, *module_args, **module_kwargs):
        self.typename, self.module_args, self.module_kwargs = typename, module_args, module_kwargs

    def build(self, log=False):
        return self.typename(*self.module_args, **self.module_kwargs)

    def __repr__(self):
        return f"LayerSpec({self.typename.__name__})"


class TiedLayerSpec(LayerSpec):
    def __init__(self, key, typename, *module_args, forward_fn=None, tied_weight_attr="weight", **module_kwargs):
        super().__init__(typename, *module_args, **module_kwargs)
        self.key, self.forward_fn, self.tied_weight_attr = key, forward_fn, tied_weight_attr


def _balanced_bounds(weights, parts):
    """Contiguous partition of `weights` into `parts` pieces minimising the heaviest piece."""
    n = len(weights)
    prefix = [0]
    for w in weights:
        prefix.append(prefix[-1] + w)

    def fits(cap):
        bounds, start = [0], 0
        for _ in range(parts):
            end = start
            while end < n and prefix[end + 1] - prefix[start] <= cap:
                end += 1
            bounds.append(end)
            start = end
        return bounds if bounds[-1] == n else None

    lo, hi = max(weights) if weights else 0, prefix[-1]
    best = fits(hi)
    while lo < hi:
        mid = (lo + hi) // 2
        b = fits(mid)
        if b:
            best, hi = b, mid
        else:
            lo = mid + 1
    return best


class PipelineModule(torch.nn.Module):
    def __init__(self, layers, num_stages=None, topology=None, loss_fn=None, seed_layers=False, seed_fn=None,
                 base_seed=1234, partition_method="parameters", activation_checkpoint_interval=0,
                 activation_checkpoint_func=checkpointing.checkpoint, checkpointable_layers=None):
        torch.nn.Module.__init__(self)
        self._layer_specs = list(layers)
        self.loss_fn = loss_fn
        self._topo = topology
        self.activation_checkpoint_interval = activation_checkpoint_interval
        self.activation_checkpoint_func = activation_checkpoint_func
        self.checkpointable_layers = checkpointable_layers
        self.global_rank = dist.get_rank() if dist.is_initialized() else 0
        self.num_stages = topology.get_dim("pipe") if topology is not None else (num_stages or 1)
        self.stage_id = topology.get_coord(self.global_rank).pipe if topology is not None else 0
        self.forward_funcs, self.fwd_map = [], {}
        self.tied_modules = torch.nn.ModuleDict()
        self.tied_weight_attrs = {}
        self._partition(partition_method)
        self._build()

    # ---- partitioning
    def _partition(self, method):
        n, parts = len(self._layer_specs), self.num_stages
        method = (method or "parameters").lower()
        if method == "uniform":
            w = [1] * n
        elif method.startswith("type:"):
            pat = re.compile(method.split(":", 1)[1], re.IGNORECASE)
            w = [1 if pat.search(self._name_of(s)) else 0 for s in self._layer_specs]
        else:
            raise NotImplementedError(f"partition method {method} (stand-in supports uniform and type:regex)")
        self.parts = _balanced_bounds(w, parts)
        self._local_start, self._local_stop = self.parts[self.stage_id], self.parts[self.stage_id + 1]

    @staticmethod
    def _name_of(spec):
        if isinstance(spec, LayerSpec):
            return spec.typename.__name__
        if isinstance(spec, torch.nn.Module):
            return spec.__class__.__name__
        return getattr(spec, "__name__", "fn")

    def _build(self):
        for idx in range(self._local_start, self._local_stop):
            spec = self._layer_specs[idx]
            if isinstance(spec, torch.nn.Module):
                self.forward_funcs.append(spec)
                self.fwd_map[str(idx)] = len(self.forward_funcs) - 1
                self.add_module(str(idx), spec)
            elif isinstance(spec, TiedLayerSpec):
                if spec.key not in self.tied_modules:
                    self.tied_modules[spec.key] = spec.build()
                    self.tied_weight_attrs[spec.key] = spec.tied_weight_attr
                mod = self.tied_modules[spec.key]
                if spec.forward_fn is None:
                    self.forward_funcs.append(mod)
                else:
                    self.forward_funcs.append(_Bound(spec.forward_fn, mod))
            elif isinstance(spec, LayerSpec):
                mod = spec.build()
                self.forward_funcs.append(mod)
                self.fwd_map[str(idx)] = len(self.forward_funcs) - 1
                self.add_module(str(idx), mod)
            else:
                self.forward_funcs.append(spec)
        for p in self.parameters():
            p.ds_pipe_replicated = False

    # ---- tied weights: which stages hold each key
    def tied_stage_sets(self):
        owners = collections.defaultdict(set)
        for stage in range(self.num_stages):
            for idx in range(self.parts[stage], self.parts[stage + 1]):
                s = self._layer_specs[idx]
                if isinstance(s, TiedLayerSpec):
                    owners[s.key].add(stage)
        return {k: sorted(v) for k, v in owners.items()}

    def topology(self):
        return self._topo

    def mpu(self):
        return None

    def num_pipeline_stages(self):
        return self.num_stages

    def _is_checkpointable(self, funcs):
        if self.checkpointable_layers is not None:
            return all(f.__class__.__name__ in self.checkpointable_layers for f in funcs)
        params = [f.parameters() for f in funcs if isinstance(f, torch.nn.Module)]
        return any(len(list(p)) > 0 for p in params)

    def forward(self, forward_input):
        def exec_range(start, end):
            def run(*inputs):
                if len(inputs) == 1:
                    inputs = inputs[0]
                for layer in self.forward_funcs[start:end]:
                    inputs = layer(inputs)
                return inputs
            return run

        n = len(self.forward_funcs)
        if self.activation_checkpoint_interval == 0:
            return exec_range(0, n)(forward_input)
        x = forward_input
        for start in range(0, n, self.activation_checkpoint_interval):
            end = min(start + self.activation_checkpoint_interval, n)
            if not isinstance(x, tuple):
                x = (x,)
            if self._is_checkpointable(self.forward_funcs[start:end]):
                x = self.activation_checkpoint_func(exec_range(start, end), *x)
            else:
                x = exec_range(start, end)(*x)
        return x


class _Bound:
    def __init__(self, fn, mod):
        self.fn, self.mod = fn, mod

    def __call__(self, x):
        return self.fn(self.mod, x)
