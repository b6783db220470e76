"""Mixed-precision optimizer over contiguous flat buffers with ZeRO-1 style sharding.

What DeepSpeed's ``BF16_Optimizer`` / ``FP16_Optimizer`` / ``DeepSpeedZeroOptimizer`` stage 1-2 provide
to the reference (``megatron/training.py:1278-1288``, config block ``zero_optimization``), re-designed
around three flat buffers per parameter bucket:

* ``flat_param``  (model dtype)  -- every parameter is a *view* into it;
* ``flat_grad``   (fp32)         -- every ``param.main_grad`` is a view into it; weight-gradient GEMMs
  accumulate into it from their epilogue, other gradients are added by a post-accumulate hook;
* per data-parallel rank a *shard* ``[lo, hi)`` of the bucket with fp32 master weights and the inner
  optimizer's state (e.g. Adam ``m``/``v``).

One step at a gradient-accumulation boundary:

1. ``reduce``: ZeRO >= 1 reduce-scatters ``flat_grad`` over the data-parallel group so each rank owns the
   summed gradient of its shard (stage 0 all-reduces);
2. the global gradient norm is the root of (sum of squares of every shard), all-reduced over the DP,
   TP and PP groups, counting tensor-parallel-replicated parameters once; it doubles as the fp16
   overflow test;
3. the inner optimizer updates the fp32 shard; un-scaling (loss scale, clip factor) is a scalar
   multiplier consumed by the update kernel, and the fused Adam kernel also writes the model-dtype
   copy straight into ``flat_param``;
4. ZeRO >= 1 all-gathers ``flat_param`` in place.

ZeRO stage 2 (``zero_optimization.stage: 2``) additionally partitions the gradients: ``flat_grad`` becomes a
transient per-bucket buffer that is allocated when a micro-batch's first gradient for the bucket appears
(``ops.linear.main_grad_of``), reduce-scattered into a persistent fp32 accumulator of shard size as soon as all of the
bucket's gradients of that micro-batch exist, and released -- so between buckets only ``1 / dp`` of the gradients
is resident, at the price of one reduce-scatter per micro-batch instead of one per step (DeepSpeed's trade as well;
like there it excludes pipeline parallelism).  Stage 3 additionally partitions the parameters (``engine/zero3.py``).

A bucket is keyed by (optimizer param group, communication group) so MoE expert parameters, which
are data-parallel only over the expert-data-parallel group, live in their own bucket.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..parallel import mpu
from .loss_scaler import DynamicLossScaler, StaticLossScaler

_ALIGN = 128  # elements; keeps every shard boundary 256-byte aligned for bf16 and 512 for fp32


# signal-pad slots of the peer-memory traffic (one block of 8 rank slots each) and the bound of its waits
_READY, _DONE, _GATHERED = 0, 8, 16
_WAIT_ROUNDS = 60      # x about two seconds


_same_host = {}


def peer_traffic_enabled(group=None) -> bool:
    """ZeRO-1 reduce-scatter / all-gather through peer memory instead of NCCL.  ``NEOX_ZERO_PEER=0`` / ``1`` forces
    it; by default it is used when every rank of the communication group runs on this host (one NVLink domain: the
    buffers are exchanged as CUDA IPC handles) under the NCCL backend."""
    mode = os.environ.get("NEOX_ZERO_PEER", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    if not (torch.cuda.is_available() and dist.is_available() and dist.is_initialized()):
        return False
    if dist.get_backend(group) != "nccl":
        return False
    key = id(group)
    if key not in _same_host:
        import socket
        names = [None] * dist.get_world_size(group)
        dist.all_gather_object(names, socket.gethostname(), group=group)
        _same_host[key] = len(set(names)) == 1
    return _same_host[key]


def _lib():
    from ..ops import native
    return native.lib()


def _check(rc, what):
    from ..ops import native
    native.check(rc, what)


def _cur_stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class _StreamWork:
    """``wait()`` makes the current stream wait for everything enqueued so far on ``stream`` (the handle of a
    reduction that was launched as kernels rather than as an NCCL call)."""

    def __init__(self, stream):
        self.event = torch.cuda.Event()
        self.event.record(stream)

    def wait(self):
        torch.cuda.current_stream().wait_event(self.event)


def _pad_to(n, m):
    return (n + m - 1) // m * m


class Bucket:
    """One contiguous (param, grad, master-shard) triple."""

    def __init__(self, params, group_opts, comm_group, comm_world, comm_rank, model_dtype, device, sharded,
                 grad_dtype=torch.float32, partition_grads=False, offload=False):
        # tensor-parallel-replicated parameters first: their squared norm is counted on TP rank 0 only
        rep = [p for p in params if not getattr(p, "model_parallel", False)]
        shd = [p for p in params if getattr(p, "model_parallel", False)]
        self.params = rep + shd
        self.opts = group_opts
        self.comm_group, self.world, self.rank = comm_group, comm_world, comm_rank
        self.sharded = sharded and comm_world > 1
        # ZeRO stage 2: the full-size gradient buffer is transient -- allocated when the first gradient of a
        # micro-batch arrives, reduce-scattered into the persistent fp32 shard accumulator as soon as the bucket is
        # complete, and released; between those moments only 1 / world of the gradients is held
        self.partition_grads = bool(partition_grads) and self.sharded
        offs, off = [], 0
        for p in self.params:
            offs.append(off)
            off += _pad_to(p.numel(), 8)
        self.rep_end = offs[len(rep)] if shd else off
        if not shd:
            self.rep_end = off
        self.numel = off
        self.padded = _pad_to(max(off, 1), _ALIGN * max(comm_world, 1))
        self.offsets = offs
        self.peer = (self.sharded and not self.partition_grads and torch.device(device).type == "cuda"
                     and comm_world <= 8
                     and grad_dtype == torch.float32
                     and model_dtype in (torch.bfloat16, torch.float16, torch.float32)
                     and peer_traffic_enabled(comm_group))
        if self.peer:
            # both flat buffers in symmetric memory: the owner of a shard reads it from every rank's gradient
            # buffer, and writes its updated shard into every rank's parameter buffer (csrc/comm_gemm_sm100.cu)
            from ..parallel import symm_mem as S
            esize = torch.empty((), dtype=model_dtype).element_size()
            self._sym_p = S.SymmBuffer(self.padded * esize, comm_group)
            self._sym_g = S.SymmBuffer(self.padded * 4, comm_group)
            self._pad = S.SignalPad(comm_group)
            self.flat_param = self._sym_p.tensor((self.padded,), model_dtype)
            self.flat_grad = self._sym_g.tensor((self.padded,), torch.float32)
            self._ctr = torch.zeros(4, dtype=torch.int32, device=device)
            self._esize = esize
            self.epoch = 0                  # one reduction (and at most one gather) per epoch
            self._gather_epoch = 0          # epoch of a gather that has not been waited for yet
        else:
            self.flat_param = torch.zeros(self.padded, dtype=model_dtype, device=device)
            self.flat_grad = None if self.partition_grads else torch.zeros(self.padded, dtype=grad_dtype, device=device)
        self.device, self.grad_dtype = device, grad_dtype
        for p, o in zip(self.params, offs):
            view = self.flat_param[o:o + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = None if self.partition_grads else self.flat_grad[o:o + p.numel()].view(p.shape)
            p.grad_in_main = False
        shard = self.padded // self.world if self.sharded else self.padded
        self.lo = shard * self.rank if self.sharded else 0
        self.hi = self.lo + shard
        self.mixed = model_dtype != torch.float32
        # optimizer-state offload (ZeRO-Offload): the fp32 master shard and the optimizer states live in host memory
        # (pinned when the model is on a GPU); each step copies the reduced gradient shard down, runs the host
        # optimizer, and copies the updated shard -- already rounded to bf16 by the host kernel when the model is
        # bf16 -- back up into the parameter buffer
        self.offload = bool(offload)
        self.host_grad = self.host_out = None
        if self.offload:
            pin = torch.device(device).type == "cuda"
            host = lambda dtype: torch.empty(shard, dtype=dtype, device="cpu", pin_memory=pin)
            m = host(torch.float32)
            m.copy_(self.flat_param[self.lo:self.hi])
            self.master = torch.nn.Parameter(m)
            self.host_grad = host(torch.float32)
            self.host_out = host(torch.bfloat16) if model_dtype == torch.bfloat16 else None
            self.master.model_out = self.host_out
        elif self.mixed:
            self.master = torch.nn.Parameter(self.flat_param[self.lo:self.hi].float().clone())
            self.master.model_out = self.flat_param[self.lo:self.hi]
        else:
            self.master = torch.nn.Parameter(self.flat_param[self.lo:self.hi])   # a view: updated in place
            self.master.model_out = None
        self.grad_acc = torch.zeros(shard, dtype=torch.float32, device=device) if self.partition_grads else None
        self.partition_params = False      # ZeRO stage 3 (engine/zero3.py): flat_param is transient, param_shard persistent
        self.param_shard = None
        self._partition_stream = None
        # overlap bookkeeping (see FlatMixedPrecisionOptimizer.arm_overlap)
        self.n_expected = len(self.params)
        self.ready = set()             # ids of the parameters whose gradient has been reported this backward
        self.never_early = any(getattr(p, "late_grad_sync", False) for p in self.params)
        self.pending_reduce = None
        self.pending_gather = None

    # ---- ZeRO stage 2: transient full-size gradients
    def ensure_grad_buffer(self):
        """Allocate (zeroed) the full-size gradient buffer of this micro-batch and point ``main_grad`` into it."""
        if not self.partition_grads or self.flat_grad is not None:
            return
        self.flat_grad = torch.zeros(self.padded, dtype=self.grad_dtype, device=self.device)
        for p, o in zip(self.params, self.offsets):
            p.main_grad = self.flat_grad[o:o + p.numel()].view(p.shape)

    def reduce_and_release(self, stream=None):
        """Reduce-scatter this micro-batch's gradients into the shard accumulator and give the buffer back."""
        if not self.partition_grads or self.flat_grad is None:
            return
        flat = self.flat_grad
        self.flat_grad = None
        for p in self.params:
            p.main_grad = None
            p.grad_in_main = False
        self.ready = set()
        if stream is not None and flat.is_cuda:
            stream.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(stream):
                tmp = torch.empty_like(self.grad_acc)
                dist.reduce_scatter_tensor(tmp, flat, group=self.comm_group)
                self.grad_acc.add_(tmp)
            flat.record_stream(stream)         # the allocator reuses the buffer only after the collective
            tmp.record_stream(stream)
            self._partition_stream = stream
        else:
            tmp = torch.empty_like(self.grad_acc)
            dist.reduce_scatter_tensor(tmp, flat, group=self.comm_group)
            self.grad_acc.add_(tmp)

    def grad_of_shard(self):
        """This rank's reduced fp32 gradient shard (view of the flat buffer, or the stage-2 accumulator)."""
        if self.partition_grads:
            if self._partition_stream is not None:
                torch.cuda.current_stream().wait_stream(self._partition_stream)
                self._partition_stream = None
            return self.grad_acc
        return self.flat_grad[self.lo:self.hi]

    # ---- gradients
    def reduce_grads(self, average_factor):
        """Sum gradients over the communication group (and divide by ``average_factor``)."""
        if self.partition_grads:
            self.reduce_and_release()
            if average_factor != 1.0:
                self.grad_acc.div_(average_factor)
            return
        if self.world > 1:
            if self.peer:
                self._peer_reduce(1.0 / average_factor)
                return
            if average_factor != 1.0:
                self.flat_grad.div_(average_factor)
            if self.sharded:
                dist.reduce_scatter_tensor(self.flat_grad[self.lo:self.hi], self.flat_grad, group=self.comm_group)
            else:
                dist.all_reduce(self.flat_grad, group=self.comm_group)

    def reduce_grads_async(self, stream):
        """Start the gradient reduction of this bucket on ``stream`` (ordered after everything launched so far on the
        current stream); ``finish_reduce`` makes the current stream wait for it."""
        if self.world <= 1 or self.pending_reduce is not None:
            return
        if self.partition_grads:
            self.reduce_and_release(stream)
            return
        if stream is not None:
            stream.wait_stream(torch.cuda.current_stream())
            ctx = torch.cuda.stream(stream)
        else:
            from contextlib import nullcontext
            ctx = nullcontext()
        with ctx:
            if self.peer:
                self._peer_reduce(1.0)
                self.pending_reduce = _StreamWork(stream)
            elif self.sharded:
                dst = self.flat_grad[self.lo:self.hi]
                if not dst.is_cuda:
                    self._rs_tmp = torch.empty_like(dst)
                    dst = self._rs_tmp
                self.pending_reduce = dist.reduce_scatter_tensor(dst, self.flat_grad, group=self.comm_group,
                                                                 async_op=True)
            else:
                self.pending_reduce = dist.all_reduce(self.flat_grad, group=self.comm_group, async_op=True)

    def finish_reduce(self):
        """Wait for an early reduction, or do it now if none was started.  Returns True if it had been overlapped."""
        if self.partition_grads:
            self.reduce_and_release()
            return False
        if self.pending_reduce is None:
            self.reduce_grads(1.0)
            return False
        self.pending_reduce.wait()
        self.pending_reduce = None
        tmp = getattr(self, "_rs_tmp", None)
        if tmp is not None:
            self.flat_grad[self.lo:self.hi].copy_(tmp)
            self._rs_tmp = None
        return True

    def gather_params_async(self, stream):
        """Start the all-gather of the updated parameter shards; ``wait_params`` is called before their first use."""
        if not self.sharded or self.partition_params:
            return
        if stream is None or not self.flat_param.is_cuda:
            self.gather_params()
            return
        stream.wait_stream(torch.cuda.current_stream())
        if self.peer:
            with torch.cuda.stream(stream):
                self._peer_push()
            return
        with torch.cuda.stream(stream):
            self.pending_gather = dist.all_gather_into_tensor(self.flat_param, self.flat_param[self.lo:self.hi],
                                                              group=self.comm_group, async_op=True)

    def wait_params(self):
        if self.peer:
            if self._gather_epoch:
                # the peers' shards of that epoch have landed in this rank's parameter buffer
                rc = _lib().neox_wait_flags_long(self._pad.word(_GATHERED), ctypes.c_uint(self._gather_epoch),
                                                 self.world, self.rank, _WAIT_ROUNDS, _cur_stream())
                _check(rc, "neox_wait_flags_long")
                self._gather_epoch = 0
            return
        if self.pending_gather is not None:
            self.pending_gather.wait()
            self.pending_gather = None

    def shard_sq_norm(self, tp_rank):
        """Squared L2 norm of this rank's gradient shard, counting TP-replicated entries on TP rank 0 only.
        On CUDA one reduction kernel per segment accumulates into a scalar (no temporaries)."""
        g = self.grad_of_shard()
        rep_hi = min(max(self.rep_end, self.lo), self.hi) - self.lo
        segs = []
        if rep_hi > 0 and tp_rank == 0:
            segs.append(g[:rep_hi])
        if rep_hi < g.numel():
            segs.append(g[rep_hi:])
        total = torch.zeros((), dtype=torch.float32, device=g.device)
        for seg in segs:
            if seg.is_cuda and seg.dtype == torch.float32:
                from ..ops import native
                import ctypes
                rc = native.lib().neox_sumsq_f32(native.ptr(seg), ctypes.c_longlong(seg.numel()), native.ptr(total),
                                                 ctypes.c_void_p(native.stream_ptr()))
                native.check(rc, "neox_sumsq_f32")
            else:
                total = total + torch.linalg.vector_norm(seg.float()) ** 2
        return total

    def gather_params(self):
        if self.partition_params:
            return          # stage 3: parameters are gathered per layer, right before use
        if self.peer:
            self._peer_push()
            self.wait_params()
            return
        if self.sharded:
            src = self.flat_param[self.lo:self.hi]
            if not src.is_cuda:
                src = src.clone()      # gloo does not define the aliased (in-place) form
            dist.all_gather_into_tensor(self.flat_param, src, group=self.comm_group)

    # ---- peer-memory forms (launched on the current stream)
    def _peer_reduce(self, scale):
        """This rank's shard <- scale * sum over ranks (rank order, fp32), read from the peers' gradient buffers."""
        L = _lib()
        self.epoch += 1
        e = ctypes.c_uint(self.epoch)
        st = _cur_stream()
        # "my gradients of this bucket are final" to every rank, then wait for everybody else's
        _check(L.neox_symm_release(None, 0, self._pad.c_ptrs, self.world, self.rank, _READY, e, st), "neox_symm_release")
        _check(L.neox_wait_flags_long(self._pad.word(_READY), e, self.world, self.rank, _WAIT_ROUNDS, st),
               "neox_wait_flags_long")
        rc = L.neox_zero_reduce_scatter(self._sym_g.c_ptrs, ctypes.c_ulonglong(self.lo),
                                        ctypes.c_ulonglong(self.hi - self.lo), ctypes.c_float(scale),
                                        self._pad.word(_READY), e, self._pad.c_ptrs, self.world, self.rank, _DONE,
                                        ctypes.c_void_p(self._ctr.data_ptr()), st)
        _check(rc, "neox_zero_reduce_scatter")

    def _peer_push(self):
        """Write this rank's updated parameter shard into every rank's parameter buffer."""
        rc = _lib().neox_zero_param_push(self._sym_p.c_ptrs, ctypes.c_ulonglong(self.lo * self._esize),
                                         ctypes.c_ulonglong((self.hi - self.lo) * self._esize), self._pad.c_ptrs,
                                         self.world, self.rank, _GATHERED, ctypes.c_uint(self.epoch),
                                         ctypes.c_void_p(self._ctr.data_ptr() + 4), _cur_stream())
        _check(rc, "neox_zero_param_push")
        self._gather_epoch = self.epoch

    def zero_grad(self):
        if self.peer and self.epoch:
            # every rank has finished reading this rank's gradients of the last reduction
            rc = _lib().neox_wait_flags_long(self._pad.word(_DONE), ctypes.c_uint(self.epoch), self.world, self.rank,
                                             _WAIT_ROUNDS, _cur_stream())
            _check(rc, "neox_wait_flags_long")
        if self.partition_grads:
            self.grad_of_shard().zero_()
            self.flat_grad = None
            self.ready = set()
            for p in self.params:
                p.grad, p.main_grad, p.grad_in_main = None, None, False
            return
        self.flat_grad.zero_()
        for p in self.params:
            p.grad = None
            p.grad_in_main = False


class FlatMixedPrecisionOptimizer:
    """See module docstring.  ``inner_cls(param_groups, **defaults)`` is any element-wise
    ``torch.optim.Optimizer`` (fused Adam, Lion, SGD, MADGRAD ...): it sees one flat fp32 parameter per
    bucket whose ``.grad`` is the reduced gradient shard."""

    def __init__(self, param_groups, inner_cls, inner_defaults, model_dtype, zero_stage=0, clip_grad=0.0,
                 fp16_cfg=None, gradient_predivide_factor=1.0, prescale_gradients=False, device=None,
                 overlap_comm=False, reduce_bucket_size=None, offload_optimizer=False,
                 partition_params_at_build=False, offload_param=False):
        """``overlap_comm``: split every parameter group into buckets of at most ``reduce_bucket_size`` elements (in
        model order), start each bucket's data-parallel gradient reduction on a side stream as soon as the LAST
        micro-batch's backward has produced all of its gradients, and all-gather the updated parameter shards
        asynchronously, each layer waiting for its own bucket in a forward pre-hook
        (``zero_optimization.overlap_comm`` / ``reduce_bucket_size`` of the DeepSpeed ZeRO-1/2 config the reference
        passes through).  ``offload_optimizer``: keep the fp32 masters and the optimizer states in host memory and
        run ``inner_cls`` there (``zero_optimization.cpu_offload`` / ``offload_optimizer.device: cpu``); ``inner_cls``
        must accept host tensors (``optim.cpu_adam.CPUAdam``, ``torch.optim.Adam`` ...).
        ``partition_params_at_build`` (stage 3): every bucket is reduced to this rank's shard as soon as it has been
        laid out, before the next one is built, so a model whose layers were parked in host memory while it was
        constructed (``engine.pipe_module.built_through``) never exists in full on the device: the peak is the
        shards plus one bucket.  ``device``: where the buckets live when the parameters are still elsewhere."""
        self.zero_stage = int(zero_stage or 0)
        self.offload_optimizer = bool(offload_optimizer)
        self.overlap_comm = bool(overlap_comm)
        self._armed = False
        self._comm_stream = None
        self.overlapped_reductions = 0
        self.clip_grad = float(clip_grad or 0.0)
        self.model_dtype = model_dtype
        self.overflow = False
        self.skipped_steps = 0
        self._global_grad_norm = 0.0
        self.buckets: list[Bucket] = []
        self.max_resident_at_build = 0      # full-size sharded buckets alive at once while the buckets were laid out
        dp_group, dp_world, dp_rank = mpu.get_data_parallel_group(), mpu.get_data_parallel_world_size(), \
            mpu.get_data_parallel_rank()
        inner_groups = []
        for gi, grp in enumerate(param_groups):
            params = [p for p in grp["params"] if p.requires_grad]
            if not params:
                continue
            opts = {k: v for k, v in grp.items() if k != "params"}
            dense = [p for p in params if not getattr(p, "expert_parallel", False)]
            expert = [p for p in params if getattr(p, "expert_parallel", False)]
            for plist, (cg, cw, cr) in ((dense, (dp_group, dp_world, dp_rank)),
                                        (expert, (mpu.get_expert_data_parallel_group(),
                                                  mpu.get_expert_data_parallel_world_size(),
                                                  _rank_in(mpu.get_expert_data_parallel_group())))):
                if not plist:
                    continue
                dev = device or plist[0].device
                chunks = [plist]
                if (self.overlap_comm or self.zero_stage >= 2) and cw > 1 and reduce_bucket_size:
                    # gradients that are rewritten after backward (norms under sequence parallelism, weights tied
                    # across layers or pipeline stages) get a bucket of their own that is reduced in step()
                    late = [p for p in plist if getattr(p, "late_grad_sync", False)]
                    chunks, cur, n = ([late] if late else []), [], 0
                    for p in plist:
                        if getattr(p, "late_grad_sync", False):
                            continue
                        if cur and n + p.numel() > reduce_bucket_size:
                            chunks.append(cur)
                            cur, n = [], 0
                        cur.append(p)
                        n += p.numel()
                    if cur:
                        chunks.append(cur)
                for chunk in chunks:
                    b = Bucket(chunk, opts, cg, cw, cr, model_dtype, dev, sharded=self.zero_stage >= 1,
                               partition_grads=self.zero_stage >= 2, offload=self.offload_optimizer)
                    self.buckets.append(b)
                    inner_groups.append({"params": [b.master], **opts})
                    if partition_params_at_build and b.partition_grads:
                        from .zero3 import partition_bucket
                        self.max_resident_at_build = max(self.max_resident_at_build,
                                                         sum(x.flat_param is not None and x.partition_grads
                                                             for x in self.buckets))
                        partition_bucket(b, offload_param)
        self.optimizer = inner_cls(inner_groups, **inner_defaults)
        self.param_groups = self.optimizer.param_groups
        self.dp_world = dp_world
        if model_dtype == torch.float16:
            cfg = fp16_cfg or {}
            if cfg.get("loss_scale", 0) in (0, None):
                self.loss_scaler = DynamicLossScaler(init_scale=2 ** cfg.get("initial_scale_power", 16),
                                                     scale_window=cfg.get("loss_scale_window", 1000),
                                                     min_scale=cfg.get("min_loss_scale", 1),
                                                     hysteresis=cfg.get("hysteresis", 2))
            else:
                self.loss_scaler = StaticLossScaler(cfg["loss_scale"])
        else:
            self.loss_scaler = StaticLossScaler(1.0)
        self._install_grad_hooks()

    # ------------------------------------------------------------------ hooks
    def _install_grad_hooks(self):
        """Fold autograd-produced ``.grad`` tensors (biases, norms, embeddings ...) into ``main_grad``."""
        def make(p, bucket):
            def hook(param):
                if param.grad is not None:
                    bucket.ensure_grad_buffer()
                    param.main_grad.add_(param.grad.to(param.main_grad.dtype))
                    param.grad = None
                    self._on_grad_ready(bucket, param)
            return hook
        self._hooks = []
        for b in self.buckets:
            for p in b.params:
                p._bucket = b
                # kernels that accumulate straight into main_grad report here (ops.linear.notify_grad_ready)
                p._grad_ready = (lambda bucket=b, param=p: self._on_grad_ready(bucket, param))
                self._hooks.append(p.register_post_accumulate_grad_hook(make(p, b)))

    # ------------------------------------------------------------------ communication overlap
    def _stream(self):
        if self._comm_stream is None and torch.cuda.is_available():
            self._comm_stream = torch.cuda.Stream()
        return self._comm_stream

    def arm_overlap(self):
        """Call right before the backward pass of the last micro-batch of a step: from now on a bucket whose
        parameters have all reported their gradient is reduced immediately, concurrently with the rest of backward."""
        if not self.overlap_comm:
            return
        self._armed = True
        for b in self.buckets:
            b.ready = set()

    def _on_grad_ready(self, bucket, param):
        """A parameter may report more than once per backward (a weight with several uses): readiness is counted
        per distinct parameter, and a bucket holding a gradient that is still rewritten after backward never fires."""
        if bucket.partition_grads:
            # stage 2: every micro-batch -- the buffer goes back as soon as the bucket's gradients are complete
            if bucket.never_early:
                return
            bucket.ready.add(id(param))
            if len(bucket.ready) == bucket.n_expected:
                bucket.reduce_and_release(self._stream() if self.overlap_comm else None)
            return
        if not self._armed or bucket.world <= 1 or bucket.never_early or self._local_grads():
            return
        bucket.ready.add(id(param))
        if len(bucket.ready) == bucket.n_expected:
            bucket.reduce_grads_async(self._stream())

    @property
    def partition_grads(self) -> bool:
        return any(b.partition_grads for b in self.buckets)

    param_partitioner = None

    def enable_param_partitioning(self, model, offload_param=False):
        """ZeRO stage 3: keep only this rank's shard of every parameter bucket between uses (engine/zero3.py)."""
        from .zero3 import ParamPartitioner
        if self.param_partitioner is None and self.partition_grads:
            self.param_partitioner = ParamPartitioner(self, offload_param=offload_param).install(model)
        return self.param_partitioner

    def end_micro_batch(self):
        """Stage 2, after the backward pass of every micro-batch (and after the gradient fix-ups that follow it):
        reduce and release whatever is still held -- buckets with late-synchronised or unused parameters."""
        for b in self.buckets:
            if b.partition_grads:
                b.reduce_and_release(self._stream() if self.overlap_comm else None)

    def install_param_wait_hooks(self, module):
        """Forward pre-hooks on the direct children of ``module`` (the layers): a layer waits for the all-gather of
        exactly the buckets that hold its parameters, so the gather of later layers overlaps earlier layers' forward."""
        if not self.overlap_comm:
            return
        for child in module.children():
            if isinstance(child, (torch.nn.ModuleDict, torch.nn.ModuleList, torch.nn.Sequential)):
                self.install_param_wait_hooks(child)
                continue
            buckets = []
            for p in child.parameters():
                b = getattr(p, "_bucket", None)
                if b is not None and b.sharded and all(b is not x for x in buckets):
                    buckets.append(b)
            if buckets:
                child.register_forward_pre_hook(lambda m, a, bs=tuple(buckets): [b.wait_params() for b in bs] and None)

    # ------------------------------------------------------------------ properties the training loop reads
    @property
    def cur_scale(self):
        return self.loss_scaler.cur_scale

    @property
    def loss_scale(self):
        return self.loss_scaler.cur_scale

    def scale_loss(self, loss):
        s = self.loss_scaler.cur_scale
        return loss * s if s != 1.0 else loss

    def zero_grad(self, set_to_none=True):
        for b in self.buckets:
            b.zero_grad()

    # ------------------------------------------------------------------ the step
    def _local_grads(self) -> bool:
        """The inner optimizer communicates by itself (1-bit Adam after its warm-up: compressed momentum instead of
        gradients), so the data-parallel gradient reduction is skipped and every rank steps on its local gradients."""
        return bool(getattr(self.optimizer, "compression_active", False)) and self.dp_world > 1

    def global_grad_norm(self, local_grads=False):
        tp_rank = mpu.get_model_parallel_rank()
        dev = self.buckets[0].master.device if self.buckets else torch.device("cpu")
        total = torch.zeros((), dtype=torch.float32, device=dev)
        expert_parallel = mpu.get_expert_parallel_world_size() > 1
        across_dp = torch.zeros((), dtype=torch.float32, device=dev)   # part that differs between DP ranks
        need_dp = False
        for b in self.buckets:
            sq = b.shard_sq_norm(tp_rank)
            b._sq = sq
            is_expert = b.comm_group is not mpu.get_data_parallel_group() and expert_parallel
            if b.sharded:
                # shards partition the bucket over its group (expert buckets: a sub-group of DP, and the
                # expert-parallel ranks hold different experts, so the full DP sum counts every element once)
                across_dp = across_dp + sq
                need_dp = True
            elif is_expert:
                # unsharded expert bucket: different experts per expert-parallel rank, replicated over the
                # expert-data-parallel group -> DP sum divided by that replication
                across_dp = across_dp + sq / float(max(b.world, 1))
                need_dp = True
            elif local_grads:
                # unreduced gradients differ per rank: use the root-mean-square over the ranks, so that clipping
                # and overflow decisions are the same everywhere
                across_dp = across_dp + sq / float(max(self.dp_world, 1))
                need_dp = True
            else:
                total = total + sq      # replicated over DP: every rank already holds the full sum
        if dist.is_available() and dist.is_initialized():
            if need_dp:
                dist.all_reduce(across_dp, group=mpu.get_data_parallel_group())
            total = total + across_dp
            if mpu.get_model_parallel_world_size() > 1:
                dist.all_reduce(total, group=mpu.get_model_parallel_group())
            if mpu.get_pipe_parallel_world_size() > 1:
                dist.all_reduce(total, group=mpu.get_pipe_parallel_group())
        return total.sqrt()

    def step(self, grad_divisor=1.0):
        """Reduce, check, clip, update, gather.  ``grad_divisor``: value the summed gradients must be
        divided by in total (micro-batches x data-parallel size)."""
        self._armed = False
        local = self._local_grads()
        if local:
            assert self.zero_stage == 0, "compressed-communication optimizers need every rank to hold the whole " \
                                         "parameter: use zero_optimization.stage 0"
            grad_divisor = grad_divisor / self.dp_world     # the momentum average supplies the 1 / world
        else:
            for b in self.buckets:
                self.overlapped_reductions += int(b.finish_reduce())
        norm_t = self.global_grad_norm(local_grads=local)
        scale = self.loss_scaler.cur_scale * grad_divisor
        norm = float(norm_t) / scale
        self._global_grad_norm = norm
        overflow = not math.isfinite(norm)
        self.overflow = overflow
        self.loss_scaler.update_scale(overflow)
        if overflow:
            self.skipped_steps += 1
            self.zero_grad()
            return False
        for b in self.buckets:
            b.wait_params()          # a gather still in flight (no forward ran since the last step)
        combined = scale
        if self.clip_grad > 0.0:
            clip = norm / self.clip_grad
            if clip > 1.0:
                combined = scale * clip
        inv = 1.0 / combined
        for b, g in zip(self.buckets, self.optimizer.param_groups):
            shard_grad = b.grad_of_shard()
            if b.offload:
                b.host_grad.copy_(shard_grad, non_blocking=True)
                shard_grad = b.host_grad
            b.master.grad = shard_grad
            g["grad_scale"] = inv
        if self.offload_optimizer and torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()      # the gradient shards have landed in host memory
        if getattr(self.optimizer, "supports_grad_scale", False):
            self.optimizer.step()
        else:
            if inv != 1.0:
                for b in self.buckets:
                    b.master.grad.mul_(inv)
            self.optimizer.step()
        for b in self.buckets:
            if b.offload:
                wrote_out = b.host_out is not None and getattr(self.optimizer, "writes_host_out", False)
                (b.param_shard if b.partition_params else b.flat_param[b.lo:b.hi]).copy_(
                    b.host_out if wrote_out else b.master.data, non_blocking=True)
            elif b.mixed and not getattr(self.optimizer, "writes_model_out", False):
                (b.param_shard if b.partition_params else b.flat_param[b.lo:b.hi]).copy_(b.master.data)
            b.master.grad = None
            if self.overlap_comm:
                b.gather_params_async(self._stream())
            else:
                b.gather_params()
        if self.param_partitioner is not None:
            self.param_partitioner.release_all()      # what is resident predates this update
        self.zero_grad()
        return True

    def wait_all_params(self):
        """Make the current stream wait for every parameter all-gather still in flight (anything that reads
        parameters outside a layer's forward -- checkpoint writing, weight export -- calls this first)."""
        for b in self.buckets:
            b.wait_params()

    # ------------------------------------------------------------------ checkpointing
    def state_dict(self):
        return {
            "loss_scaler": self.loss_scaler.state_dict(),
            "skipped_steps": self.skipped_steps,
            "zero_stage": self.zero_stage,
            "partition_count": [b.world if b.sharded else 1 for b in self.buckets],
            "optimizer_state_dict": self.optimizer.state_dict(),
            "single_partition_of_fp32_groups": [b.master.data.detach().clone().cpu() for b in self.buckets],
            "bucket_numel": [b.numel for b in self.buckets],
        }

    def load_state_dict(self, sd, load_optimizer_states=True):
        self.loss_scaler.load_state_dict(sd.get("loss_scaler", {}))
        self.skipped_steps = sd.get("skipped_steps", 0)
        if load_optimizer_states and "optimizer_state_dict" in sd:
            self.optimizer.load_state_dict(sd["optimizer_state_dict"])
        for i, (b, m) in enumerate(zip(self.buckets, sd.get("single_partition_of_fp32_groups", []))):
            if m.numel() != b.master.numel():
                raise ValueError(
                    f"optimizer state of bucket {i} holds {m.numel()} master weights but this run shards the bucket "
                    f"into {b.master.numel()}: the data-parallel size or the bucket layout changed since the "
                    "checkpoint was written; reload with load_optimizer_states=False (finetune / no_load_optim) or "
                    "with the original layout")
            b.master.data.copy_(m.to(b.master.device))

    def refresh_master_from_params(self):
        """After loading module weights: re-derive the fp32 master shards from ``flat_param``."""
        self.wait_all_params()
        for b in self.buckets:
            if b.partition_params:
                # stage 3: called with the parameters resident (checkpointing wraps the load in all_resident())
                assert b.flat_param is not None, "refresh_master_from_params under ZeRO stage 3 needs resident parameters"
                b.param_shard.copy_(b.flat_param[b.lo:b.hi])
                if b.mixed or b.offload:
                    b.master.data.copy_(b.param_shard.float())
                continue
            if b.mixed or b.offload:
                b.master.data.copy_(b.flat_param[b.lo:b.hi].float())


def _rank_in(group):
    if group is None or not (dist.is_available() and dist.is_initialized()):
        return 0
    return dist.get_rank(group)
