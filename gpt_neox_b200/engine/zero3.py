"""ZeRO stage 3: parameter partitioning on top of the flat-bucket optimizer.

What ``deepspeed.zero.Init`` + ``DeepSpeedZeroOptimizer_Stage3`` give the reference when ``zero_optimization.stage``
is 3 (``megatron/training.py:958-977``), restated for the bucket layout of ``engine/flat_optimizer.py``:

* between uses a rank holds only ITS shard of every bucket's parameters (model dtype, ``bucket.param_shard``; the
  fused optimizer kernel writes its updated 16-bit copy straight there), plus the fp32 master / optimizer-state /
  gradient-accumulator shards it already had under stages 1-2;
* the full parameter buffer of a bucket is transient: right before a layer runs -- forward, recomputation, or
  backward -- the buckets holding that layer's parameters are all-gathered into a fresh buffer and every parameter's
  ``.data`` is pointed into it; buckets that neither the current nor the previous layer needs are released, and the
  released parameters keep their shape through a zero-stride placeholder (so ``numel()`` / ``shape`` stay valid).

"Layer" means a direct child of the model's layer container (the same granularity the overlapped parameter gather of
stage 1 waits at), because a layer's forward reads parameters of its sub-modules directly (fused norm heads, biases
riding in a neighbour's GEMM epilogue).  Backward without activation checkpointing is caught by a hook on the layer's
outputs, which fires when their gradient is known, i.e. just before the layer's backward.
"""
from __future__ import annotations

import contextlib

import torch
import torch.distributed as dist


def _layers(module):
    """The modules whose forward is one scheduling unit: direct children, looking through plain containers."""
    for child in module.children():
        if isinstance(child, (torch.nn.ModuleDict, torch.nn.ModuleList, torch.nn.Sequential)):
            yield from _layers(child)
        elif any(True for _ in child.parameters()):
            yield child


def _placeholder(p):
    """Stand-in for a released parameter: keeps shape / dtype / device, owns one element."""
    return torch.empty(1, dtype=p.dtype, device=p.device).expand(p.shape)


def partition_bucket(b, offload_param=False):
    """Turn a freshly built bucket into its stage-3 form: keep this rank's shard (in host memory with
    ``offload_param``), hand it to the optimizer as the place the updated 16-bit copy goes, release the full
    buffer.  Idempotent."""
    if b.partition_params:
        return
    b.param_shard = b.flat_param[b.lo:b.hi].clone()
    if offload_param:
        assert getattr(b, "offload", False), \
            "offload_param needs the optimizer states offloaded as well (zero_optimization.cpu_offload / " \
            "offload_optimizer.device: cpu)"
        host = torch.empty(b.param_shard.shape, dtype=b.param_shard.dtype, device="cpu",
                           pin_memory=b.param_shard.is_cuda)
        host.copy_(b.param_shard)
        b.param_shard = host
    if getattr(b, "offload", False):
        pass                                # host masters: the step copies the updated shard up itself
    elif b.mixed:
        b.master.model_out = b.param_shard
    else:
        b.master.data = b.param_shard       # fp32 training: the shard IS the master (same Parameter object,
        #                                     which the inner optimizer already holds)
    b.partition_params = True
    for p in b.params:
        p.data = _placeholder(p)
    b.flat_param = None


class ParamPartitioner:
    def __init__(self, optimizer, offload_param=False):
        """``offload_param``: keep the persistent 16-bit shards in (pinned) host memory as well -- the
        ``zero_optimization.offload_param`` of the reference's DeepSpeed configuration; a gather then starts with a
        host-to-device copy of the shard.  Needs the optimizer states offloaded too (the host optimizer is what
        writes the updated shard)."""
        self.opt = optimizer
        self.offload_param = bool(offload_param)
        self.buckets = [b for b in optimizer.buckets if b.partition_grads]     # the data-parallel sharded ones
        self.resident = []          # buckets whose full buffer exists, least recently used first
        self.pinned = False         # True inside all_resident(): nothing is released
        self._prev = ()
        self.gathers = 0
        for b in self.buckets:
            partition_bucket(b, self.offload_param)      # no-op for buckets partitioned while they were built

    # ------------------------------------------------------------------ gather / release
    def _gather(self, b):
        dev = torch.device(b.device)
        shard = b.param_shard if b.param_shard.device.type == dev.type else b.param_shard.to(dev, non_blocking=True)
        full = torch.empty(b.padded, dtype=shard.dtype, device=dev)
        dist.all_gather_into_tensor(full, shard, group=b.comm_group)
        b.flat_param = full
        for p, o in zip(b.params, b.offsets):
            p.data = full[o:o + p.numel()].view(p.shape)
        self.gathers += 1

    def _release(self, b):
        if b.flat_param is None:
            return
        for p in b.params:
            p.data = _placeholder(p)
        b.flat_param = None

    def acquire(self, buckets):
        """Make ``buckets`` resident; release every bucket that neither this call nor the previous one asked for."""
        for b in buckets:
            if b.flat_param is None:
                self._gather(b)
            if b in self.resident:
                self.resident.remove(b)
            self.resident.append(b)
        if not self.pinned:
            keep = set(id(b) for b in buckets) | set(id(b) for b in self._prev)
            for b in list(self.resident):
                if id(b) not in keep:
                    self._release(b)
                    self.resident.remove(b)
        self._prev = tuple(buckets)

    def release_all(self):
        for b in self.buckets:
            self._release(b)
        self.resident, self._prev = [], ()

    @contextlib.contextmanager
    def all_resident(self, write_back=False):
        """Every parameter present (checkpoint writing, weight export, ``load_state_dict``).  ``write_back``: the
        parameters were modified in there -- refresh the shards (and masters) from them before releasing."""
        self.pinned = True
        try:
            self.acquire(self.buckets)
            yield
            if write_back:
                for b in self.buckets:
                    b.param_shard.copy_(b.flat_param[b.lo:b.hi])
                    if b.mixed or getattr(b, "offload", False):
                        b.master.data.copy_(b.param_shard.float())
        finally:
            self.pinned = False
            self.release_all()

    # ------------------------------------------------------------------ hooks
    def install(self, model):
        """Forward pre-hooks (cover forward and recomputation) and output-gradient hooks (cover a backward that
        does not recompute) on every layer of ``model``."""
        by_param = {id(p): b for b in self.buckets for p in b.params}
        for layer in _layers(model):
            needed = []
            for p in layer.parameters():
                b = by_param.get(id(p))
                if b is not None and all(b is not x for x in needed):
                    needed.append(b)
            if not needed:
                continue
            needed = tuple(needed)

            def pre(module, args, needed=needed):
                self.acquire(needed)

            def post(module, args, output, needed=needed):
                outs = output if isinstance(output, (tuple, list)) else (output,)
                for o in outs:
                    if torch.is_tensor(o) and o.requires_grad:
                        o.register_hook(lambda g, needed=needed: self.acquire(needed) or g)
            layer.register_forward_pre_hook(pre)
            layer.register_forward_hook(post)
        return self
