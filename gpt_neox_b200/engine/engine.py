"""Training engines: what ``deepspeed.initialize`` returns to the reference
(``megatron/training.py:1278-1288``), written for this code base.

``NeoXEngine``      data/tensor parallel training of a sequential module: ``loss = engine(batch)``,
                    ``engine.backward(loss)``, ``engine.step()`` with gradient accumulation, loss
                    scaling, clipping, LR scheduling, ZeRO-1 sharding and checkpoint I/O.
``PipelineEngine``  adds the 1F1B pipeline executor: ``train_batch(data_iter)`` / ``eval_batch(data_iter)``
                    over ``micro_batches = gradient_accumulation_steps`` micro-batches, NCCL (or gloo)
                    point-to-point between adjacent stages with a one-time shape/dtype handshake,
                    tied-weight gradient all-reduce, loss broadcast from the last stage.

B200-first choices: the attention mask is never shipped between stages (kernels build masks
in-register); every pipeline link has one communicator per direction, sends are posted and never
waited on, and the receive for micro-batch *i+1* is posted before micro-batch *i* is computed, so
transfers run under compute (``_P2P``).
"""
from __future__ import annotations

import os
from types import SimpleNamespace

import torch
import torch.distributed as dist

from ..parallel import mpu
from ..models.utils import reduce_sequence_parallel_grads
from ..ops import fp8

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.bool, torch.uint8]


def _dist_on():
    return dist.is_available() and dist.is_initialized()


class NeoXEngine:
    def __init__(self, model, optimizer, lr_scheduler, neox_args, sp_sync_params=None):
        self.module = model
        self.optimizer = optimizer
        self.lr_scheduler = lr_scheduler
        self.neox_args = neox_args
        self.sp_sync_params = sp_sync_params or []
        self.global_steps = 0
        self.global_samples = 0
        self.skipped_steps = 0
        self.micro_steps = 0
        self.gas = max(1, int(neox_args.gradient_accumulation_steps or 1))
        self.micro_batch_size = neox_args.train_micro_batch_size_per_gpu
        self.dp_world_size = mpu.get_data_parallel_world_size()
        self.mp_world_size = mpu.get_model_parallel_world_size()
        self.store_gradients = False
        self.stored_gradients = None
        self.timers = None
        self.training = True
        self.is_pipe_parallel = False
        self.curriculum_scheduler = None
        cl = getattr(neox_args, "curriculum_learning", None)
        if cl and cl.get("enabled", True) and optimizer is not None and not getattr(neox_args, "is_pipe_parallel", False) \
                and cl.get("curriculum_type", "seqlen") == "seqlen":
            from .curriculum import CurriculumScheduler
            self.curriculum_scheduler = CurriculumScheduler(cl)
        # ``wall_clock_breakdown``: per-phase times of the engine, averaged over ``steps_per_print`` optimizer steps,
        # printed by rank 0 and left in ``timer_values`` (milliseconds per step) for the training log.  The timers
        # record CUDA events and are only resolved when they are printed, so they do not serialise the step.
        self._breakdown = bool(getattr(neox_args, "wall_clock_breakdown", False))
        self._steps_per_print = max(1, int(getattr(neox_args, "steps_per_print", None) or 10))
        self._clock = None
        self.timer_values = None
        if self._breakdown:
            from ..utils import Timers
            self._clock = Timers()

    # ------------------------------------------------------------------ mode helpers
    def train(self, mode=True):
        self.module.train(mode)
        self.training = mode
        return self

    def eval(self):
        return self.train(False)

    def __call__(self, *args, **kwargs):
        if self.training and self.curriculum_scheduler is not None:
            # sequence-length curriculum of the sequential model: the module truncates its inputs to the current
            # difficulty and records it in ``neox_args.curriculum_seqlen`` for the loss (the pipeline engine gets the
            # same through its batch function)
            kwargs["curriculum_seqlen"] = self.curriculum_scheduler.update_difficulty(self.global_steps + 1)
        with self._timed("forward" if self.training else None):
            return self.module(*args, **kwargs)

    # ------------------------------------------------------------------ wall-clock breakdown
    def wall_clock_breakdown(self):
        return self._breakdown

    def steps_per_print(self):
        return self._steps_per_print

    def _timed(self, name):
        """Context manager that accumulates the enclosed region into timer ``name`` (no-op when disabled)."""
        return _Region(self._clock(name) if (self._clock is not None and name) else None)

    def _publish_breakdown(self):
        """Called after every optimizer step: every ``steps_per_print`` steps resolve the timers."""
        if self._clock is None or self.global_steps % self._steps_per_print:
            return
        self.timer_values = {name: t.elapsed(reset=True) * 1000.0 / self._steps_per_print
                             for name, t in self._clock.timers.items()}
        if not _dist_on() or dist.get_rank() == 0:
            print("time (ms) per step | " + " | ".join(f"{k}: {v:.2f}" for k, v in self.timer_values.items()),
                  flush=True)

    def parameters(self):
        return self.module.parameters()

    def train_batch_size(self):
        return self.neox_args.train_batch_size

    def train_micro_batch_size_per_gpu(self):
        return self.micro_batch_size

    def gradient_accumulation_steps(self):
        return self.gas

    def is_gradient_accumulation_boundary(self):
        return (self.micro_steps + 1) % self.gas == 0

    def get_lr(self):
        return [g["lr"] for g in self.optimizer.param_groups] if self.optimizer else []

    def get_global_grad_norm(self):
        return getattr(self.optimizer, "_global_grad_norm", None)

    # ------------------------------------------------------------------ backward / step
    def backward(self, loss, retain_graph=False):
        """Back-propagate ``loss`` (scaled for fp16).  Gradients accumulate into fp32 ``main_grad``
        buffers; division by the number of micro-batches happens once, inside the optimizer step."""
        scaled = self.optimizer.scale_loss(loss) if self.optimizer is not None else loss
        if self.optimizer is not None and self.is_gradient_accumulation_boundary() and \
                hasattr(self.optimizer, "arm_overlap"):
            self.optimizer.arm_overlap()     # last micro-batch: reduce each bucket as soon as its gradients exist
        with self._timed("backward"):
            scaled.backward(retain_graph=retain_graph)
        if self.optimizer is not None and getattr(self.optimizer, "partition_grads", False):
            # ZeRO stage 2: gradients leave their transient full-size buffers after every micro-batch, so the
            # fix-ups that rewrite them (sequence-parallel norm gradients) run now, not at the step
            self._pre_step_grad_sync()
            self.optimizer.end_micro_batch()
        return loss

    def _pre_step_grad_sync(self):
        if self.sp_sync_params:
            reduce_sequence_parallel_grads(self.sp_sync_params)

    def step(self):
        """Optimizer step at accumulation boundaries; otherwise only counts the micro-step."""
        boundary = self.is_gradient_accumulation_boundary()
        self.micro_steps += 1
        if not boundary or self.optimizer is None:
            return
        self._take_step()

    def _take_step(self):
        with self._timed("backward_allreduce"):
            self._pre_step_grad_sync()
        if self.store_gradients:
            self.stored_gradients = [p.main_grad.detach().clone() for b in self.optimizer.buckets for p in b.params
                                     if getattr(p, "main_grad", None) is not None]
        with self._timed("step"):
            ok = self.optimizer.step(grad_divisor=float(self.gas * self.dp_world_size))
        fp8.invalidate_weight_cache()          # the fused optimizer rewrites parameters through raw pointers
        if ok:
            if self.lr_scheduler is not None:
                self.lr_scheduler.step()
        else:
            self.skipped_steps += 1
        self.global_steps += 1
        self.global_samples += self.neox_args.train_batch_size
        self._publish_breakdown()

    def zero_grad(self):
        if self.optimizer is not None:
            self.optimizer.zero_grad()

    # ------------------------------------------------------------------ checkpoint I/O (see checkpointing.py)
    def save_checkpoint(self, save_dir, tag=None, client_state=None):
        from ..checkpointing import engine_save_checkpoint
        return engine_save_checkpoint(self, save_dir, tag, client_state or {})

    def load_checkpoint(self, load_dir, tag=None, load_optimizer_states=True, load_lr_scheduler_states=True,
                        load_module_only=False, load_module_strict=True):
        from ..checkpointing import engine_load_checkpoint
        fp8.invalidate_weight_cache()
        return engine_load_checkpoint(self, load_dir, tag, load_optimizer_states, load_lr_scheduler_states,
                                      load_module_only, load_module_strict)


class _Region:
    """``with`` block around one timed phase; ``timer`` is a ``utils.Timer`` or None."""

    def __init__(self, timer):
        self.timer = timer

    def __enter__(self):
        if self.timer is not None:
            self.timer.start()

    def __exit__(self, *exc):
        if self.timer is not None:
            self.timer.stop()
        return False


# ============================================================================================== pipeline
class _Timeline:
    """Optional per-stage record of one training batch: CUDA events around every receive-wait and every forward /
    backward of the 1F1B schedule, written as JSON (``NEOX_PP_TIMELINE=<path prefix>``; the batch recorded is the
    fourth one executed, i.e. past warm-up).  The time between a ``*_wait`` mark and the following ``*_begin`` mark
    is how long the compute stream stalled for a transfer: the exposed part of the pipeline communication."""

    def __init__(self, prefix, stage):
        self.path = f"{prefix}.stage{stage}.json"
        self.marks = []

    def mark(self, name, micro_batch):
        if torch.cuda.is_available():
            e = torch.cuda.Event(enable_timing=True)
            e.record()
        else:
            import time
            e = time.perf_counter()
        self.marks.append((name, micro_batch, e))

    def dump(self):
        import json
        if torch.cuda.is_available():
            torch.cuda.synchronize()
        base = self.marks[0][2]
        rows = []
        for name, mb, e in self.marks:
            t = base.elapsed_time(e) if not isinstance(e, float) else (e - base) * 1e3
            rows.append({"event": name, "micro_batch": mb, "ms": round(t, 4)})
        with open(self.path, "w") as fh:
            json.dump(rows, fh)


class _P2P:
    """Adjacent-stage tensor exchange.

    Every (stage s -> stage s + 1) link has TWO two-rank communicators, one per direction, so that activations going
    down the pipeline and gradients coming back never share a communication stream: a send can be posted and left
    in flight while the stage computes (it completes when the neighbour posts its receive), a receive can be posted
    one micro-batch ahead, and nothing deadlocks the way unpaired sends on one communicator do.  ``wait`` is only
    called on a receive, right where its tensors are consumed; finished sends are reaped a few micro-batches later.
    The one-time (per direction) shape handshake travels over the same communicators.
    """
    _links = {}          # (lo_rank, hi_rank) -> (forward-direction group, backward-direction group)

    def __init__(self):
        self.ranks = mpu.get_pipe_parallel_ranks()
        self.stage = mpu.get_pipe_parallel_rank()
        self.group = mpu.get_pipe_parallel_group()
        self.meta = {}
        self.inflight = []          # (work, tensors) of posted sends
        topo = mpu.get_topology()
        key = (topo.pp, topo.dp, topo.mp)
        if _P2P._links.get("topology") != key:
            _P2P._links = {"topology": key}
            for pipe in topo.axis_lists("pipe"):           # every rank creates every link, in the same order
                for lo, hi in zip(pipe[:-1], pipe[1:]):
                    _P2P._links[(lo, hi)] = (dist.new_group([lo, hi]), dist.new_group([lo, hi]))
            self._connect()

    def _connect(self):
        """Bring up every communicator this rank will use -- its pipeline links in both directions and the tensor /
        pipe / data parallel groups -- with one tiny exchange each, then drain the device.  Communicator creation and
        the first connection between two peers synchronise the device; if that happened lazily in the middle of a
        step, while a receive posted ahead of time is still waiting for its sender, the two stages could wait on
        each other for ever."""
        dev = self._device()
        me = self.ranks[self.stage]
        one = torch.ones(8, device=dev)
        for delta in (-1, +1):
            if not 0 <= self.stage + delta < len(self.ranks):
                continue
            other = self.peer(delta)
            lo, hi = min(me, other), max(me, other)
            fwd, bwd = _P2P._links[(lo, hi)]
            buf = torch.zeros(8, device=dev)
            # forward-traffic communicator carries lo -> hi, the other one hi -> lo
            ops = [dist.P2POp(dist.isend if me == lo else dist.irecv, one if me == lo else buf, other, group=fwd)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
            ops = [dist.P2POp(dist.isend if me == hi else dist.irecv, one if me == hi else buf, other, group=bwd)]
            for w in dist.batch_isend_irecv(ops):
                w.wait()
        for g in (mpu.get_model_parallel_group(), mpu.get_pipe_parallel_group(), mpu.get_data_parallel_group()):
            if g is not None and dist.get_world_size(g) > 1:
                dist.all_reduce(one.clone(), group=g)
        if dev.type == "cuda":
            torch.cuda.synchronize()

    @classmethod
    def forget_links(cls):
        cls._links = {}

    def peer(self, delta):
        return self.ranks[self.stage + delta]

    def _comm(self, delta, forward_traffic):
        me, other = self.ranks[self.stage], self.peer(delta)
        return _P2P._links[(min(me, other), max(me, other))][0 if forward_traffic else 1]

    def reset(self):
        self.meta = {}

    def _device(self):
        return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")

    def _send_meta(self, tensors, dst, key, is_tuple):
        if key in self.meta:
            return
        hdr = [len(tensors), int(is_tuple)]
        for t in tensors:
            hdr += [t.dim(), _DTYPES.index(t.dtype)] + list(t.shape) + [0] * (6 - t.dim())
        buf = torch.tensor(hdr + [0] * (64 - len(hdr)), dtype=torch.int64, device=self._device())
        for w in dist.batch_isend_irecv([dist.P2POp(dist.isend, buf, dst, group=self._comm(+1, True))]):
            w.wait()
        self.meta[key] = ([(tuple(t.shape), t.dtype) for t in tensors], is_tuple)

    def _recv_meta(self, src, key):
        if key in self.meta:
            return self.meta[key]
        buf = torch.zeros(64, dtype=torch.int64, device=self._device())
        for w in dist.batch_isend_irecv([dist.P2POp(dist.irecv, buf, src, group=self._comm(-1, True))]):
            w.wait()
        h = buf.tolist()
        n, is_tuple, pos, metas = h[0], bool(h[1]), 2, []
        for _ in range(n):
            nd, dt = h[pos], h[pos + 1]
            metas.append((tuple(h[pos + 2:pos + 2 + nd]), _DTYPES[dt]))
            pos += 8
        self.meta[key] = (metas, is_tuple)
        return self.meta[key]

    def post_send(self, tensors, delta):
        """Start sending ``tensors`` to the neighbour; returns immediately (see ``reap``)."""
        if not tensors:
            return
        g = self._comm(delta, forward_traffic=delta > 0)
        ts = [t.contiguous() for t in tensors]
        works = dist.batch_isend_irecv([dist.P2POp(dist.isend, t, self.peer(delta), group=g) for t in ts])
        self.inflight.append((works, ts))
        self.reap(keep=4)

    def post_recv(self, metas, delta):
        """Start receiving tensors of the given shapes from the neighbour; ``wait`` the handle where they are used."""
        g = self._comm(delta, forward_traffic=delta < 0)
        bufs = [torch.empty(shape, dtype=dt, device=self._device()) for shape, dt in metas]
        works = dist.batch_isend_irecv([dist.P2POp(dist.irecv, b, self.peer(delta), group=g) for b in bufs]) if bufs else []
        return works, bufs

    @staticmethod
    def wait(handle):
        works, bufs = handle
        for w in works:
            w.wait()
        return bufs

    def reap(self, keep=0):
        """Release sends posted more than ``keep`` posts ago (they have long completed; ``wait`` only orders the
        current stream after them and drops the references that kept their buffers alive)."""
        while len(self.inflight) > keep:
            works, _ = self.inflight.pop(0)
            for w in works:
                w.wait()


class PipelineEngine(NeoXEngine):
    def __init__(self, model, optimizer, lr_scheduler, neox_args, sp_sync_params=None):
        super().__init__(model, optimizer, lr_scheduler, neox_args, sp_sync_params)
        if optimizer is not None and getattr(optimizer, "partition_grads", False):
            # as in the reference's engine: gradients of several micro-batches are in flight on a pipeline stage and
            # tied weights are summed after the last one, which a per-micro-batch gradient partition cannot serve
            raise ValueError("ZeRO stage 2 (gradient partitioning) cannot be combined with pipeline parallelism; "
                             "use zero_optimization.stage 1")
        self.is_pipe_parallel = True
        self.num_stages = mpu.get_pipe_parallel_world_size()
        self.stage_id = mpu.get_pipe_parallel_rank()
        self.micro_batches = self.gas
        self.batch_fn = None
        self.has_attention_mask = False
        self.p2p = _P2P() if self.num_stages > 1 else None
        self._batches_run = 0
        self.first_output_send = True
        self.pipe_recv_buf = None
        self.grid = SimpleNamespace(stage_to_global=self._stage_to_global, pipe_parallel_size=self.num_stages,
                                    data_parallel_size=self.dp_world_size, get_stage_id=lambda: self.stage_id)
        self.total_loss = None
        self.agg_loss = None
        if self.num_stages > 1 and hasattr(model, "sync_tied_weights"):
            model.sync_tied_weights()

    def _stage_to_global(self, stage_id, **kwargs):
        return mpu.get_pipe_parallel_ranks()[stage_id]

    def is_first_stage(self):
        return self.stage_id == 0

    def is_last_stage(self):
        return self.stage_id == self.num_stages - 1

    def set_batch_fn(self, fn):
        self.batch_fn = fn

    def set_has_attention_mask(self, value):
        self.has_attention_mask = value

    def reset_activation_shape(self):
        """Forget the cached message shapes (generation changes the sequence length per call)."""
        if self.p2p is not None:
            self.p2p.reset()

    # ------------------------------------------------------------------ micro-batch plumbing
    def _load_micro_batch(self, data_iter):
        if not (self.is_first_stage() or self.is_last_stage()) or data_iter is None:
            return None, None
        batch = next(data_iter)
        if self.batch_fn is not None:
            batch = self.batch_fn(batch)
        inputs, labels = batch
        return inputs, labels

    def _forward_micro(self, inputs, recv, recv_is_tuple):
        if self.is_first_stage():
            x = inputs
        elif recv_is_tuple:
            # re-attach the empty attention-mask slot that was not shipped
            x = (recv[0], None) if len(recv) == 1 else tuple(recv)
        else:
            x = recv[0] if len(recv) == 1 else tuple(recv)
        return self.module(x)

    @staticmethod
    def _tensors_of(out):
        """Tensors of a stage output that travel to the next stage (``None`` entries, such as the
        attention mask, are dropped and re-inserted on the receiver)."""
        if isinstance(out, torch.Tensor):
            return [out], False
        return [t for t in out if isinstance(t, torch.Tensor)], True

    def _exec(self, data_iter, train=True, return_logits=False, num_micro=None):
        M = num_micro if num_micro is not None else self.micro_batches
        P, s = self.num_stages, self.stage_id
        first, last = self.is_first_stage(), self.is_last_stage()
        p2p = self.p2p
        losses, logits_out = [], []
        queue = []
        warm = min(P - s - 1, M) if train else 0
        state = {"tuple": False}

        def prep(bufs):
            for b in bufs:
                if b.is_floating_point() and train:
                    b.requires_grad_(True)
            return bufs

        # The first executed batch posts every receive only when it is needed: that batch is where buffers,
        # workspaces and library handles are created (calls that may synchronise the device), which must not
        # happen while a receive posted ahead of time waits for a sender.  Later batches post receives early.
        ahead = self._batches_run > 0
        prefix = os.environ.get("NEOX_PP_TIMELINE")
        tl = _Timeline(prefix, s) if (prefix and train and self._batches_run == 3) else None
        mark = tl.mark if tl is not None else (lambda name, mb: None)

        def post_recv_fwd():
            """Post the receive of the next activation (None on the first stage)."""
            if first:
                return None

            def post():
                metas, is_tuple = p2p._recv_meta(p2p.peer(-1), "act_in")      # (a middle stage also SENDS a header)
                state["tuple"] = is_tuple
                return p2p.post_recv(metas, -1)
            return post() if ahead else post

        def take_fwd(handle):
            if handle is None:
                return None
            return prep(_P2P.wait(handle() if callable(handle) else handle))

        def send_fwd(out):
            if last:
                return
            ts, is_tuple = self._tensors_of(out)
            p2p._send_meta(ts, p2p.peer(+1), "act_out", is_tuple)
            p2p.post_send(ts, +1)

        def grad_metas(out):
            ts, _ = self._tensors_of(out)
            return [(tuple(t.shape), t.dtype) for t in ts if t.is_floating_point()]

        def post_recv_bwd(out):
            if last:
                return None
            metas = grad_metas(out)
            return p2p.post_recv(metas, +1) if ahead else (lambda: p2p.post_recv(metas, +1))

        def take_bwd(handle):
            if handle is None:
                return None
            return _P2P.wait(handle() if callable(handle) else handle)

        def send_bwd(recv):
            if first:
                return
            p2p.post_send([b.grad if b.grad is not None else torch.zeros_like(b) for b in recv if b.is_floating_point()],
                          -1)

        def fwd(recv):
            with self._timed("batch_input" if train else None):
                inputs, labels = self._load_micro_batch(data_iter)
            with self._timed("forward_microstep" if train else None):
                return fwd_compute(inputs, labels, recv)

        def fwd_compute(inputs, labels, recv):
            out = self._forward_micro(inputs, recv, state["tuple"])
            loss = None
            if last:
                if return_logits:
                    logits_out.append(out if isinstance(out, torch.Tensor) else out[0])
                if self.module.loss_fn is not None and labels is not None:
                    loss = self.module.loss_fn(out, labels)
                    losses.append(loss.detach())
            return out, loss

        bwd_count = [0]

        def bwd(out, loss, grads):
            with self._timed("backward_microstep"):
                bwd_compute(out, loss, grads)

        def bwd_compute(out, loss, grads):
            bwd_count[0] += 1
            if bwd_count[0] == M and self.optimizer is not None and hasattr(self.optimizer, "arm_overlap"):
                self.optimizer.arm_overlap()     # last micro-batch of the step on this stage
            if last:
                self.backward(loss)
            else:
                ts, _ = self._tensors_of(out)
                outs = [t for t in ts if t.is_floating_point()]
                pairs = [(o, g) for o, g in zip(outs, grads) if o.requires_grad]
                torch.autograd.backward([o for o, _ in pairs], [g for _, g in pairs])

        if not train:
            with torch.no_grad():
                nxt = post_recv_fwd() if M > 0 else None
                for i in range(M):
                    recv = take_fwd(nxt)
                    nxt = post_recv_fwd() if i + 1 < M else None       # next activation arrives during this forward
                    out, loss = fwd(recv)
                    send_fwd(out)
        else:
            # One-forward-one-backward.  The receive of the NEXT activation is posted before the current micro-batch
            # is computed and the receive of a gradient right after its forward has been sent on, so transfers
            # run under compute; sends are never waited on.
            nxt = post_recv_fwd() if M > 0 else None
            n_fwd = 0
            n_bwd = [0]

            def one_fwd():
                nonlocal nxt, n_fwd
                mark("fwd_wait", n_fwd)
                recv = take_fwd(nxt)
                n_fwd += 1
                nxt = post_recv_fwd() if n_fwd < M else None
                mark("fwd_begin", n_fwd - 1)
                out, loss = fwd(recv)
                mark("fwd_end", n_fwd - 1)
                send_fwd(out)
                queue.append((recv, out, loss, post_recv_bwd(out)))

            def one_bwd():
                r0, o0, l0, gh = queue.pop(0)          # the oldest outstanding micro-batch
                mark("bwd_wait", n_bwd[0])
                grads = take_bwd(gh)
                mark("bwd_begin", n_bwd[0])
                bwd(o0, l0, grads)
                mark("bwd_end", n_bwd[0])
                n_bwd[0] += 1
                send_bwd(r0)

            for _ in range(warm):
                one_fwd()
            for i in range(M - warm):
                one_fwd()
                one_bwd()
            while queue:
                one_bwd()
            if tl is not None:
                tl.dump()
        if p2p is not None:
            p2p.reap()
        self._batches_run += 1

        # mean loss of the micro-batches, broadcast from the last stage to the whole pipeline group
        dev = p2p._device() if p2p else (losses[0].device if losses else torch.device("cpu"))
        agg = torch.stack(losses).float().mean() if losses else torch.zeros((), device=dev)
        if P > 1:
            agg = agg.to(dev)
            dist.broadcast(agg, src=mpu.get_pipe_parallel_ranks()[-1], group=mpu.get_pipe_parallel_group())
        if self.dp_world_size > 1:
            agg = agg.clone()
            dist.all_reduce(agg, group=mpu.get_data_parallel_group())
            agg /= self.dp_world_size
        return agg, logits_out

    # ------------------------------------------------------------------ public API
    def set_curriculum_scheduler(self, scheduler):
        """The scheduler the batch function truncates sequences with: every stage follows it, so that the cached
        message shapes are dropped whenever the sequence length is about to change."""
        self._pipe_curriculum, self._pipe_difficulty = scheduler, None

    def train_batch(self, data_iter=None):
        self.module.train()
        sched = getattr(self, "_pipe_curriculum", None)
        if sched is not None:
            it = getattr(self.neox_args, "iteration", None)
            step = (it if it is not None else self.global_steps) + 1
            now = min(sched.get_difficulty(step), sched.state["max_difficulty"])
            if now != self._pipe_difficulty:
                self.reset_activation_shape()
                self._pipe_difficulty = now
        with self._timed("train_batch"):
            loss, _ = self._exec(data_iter, train=True)
        if hasattr(self.module, "allreduce_tied_weight_gradients"):
            with self._timed("backward_tied_allreduce"):
                self.module.allreduce_tied_weight_gradients()
        self.micro_steps += self.gas
        if self.optimizer is not None:
            self._take_step()
        self.agg_loss = loss
        return loss

    def eval_batch(self, data_iter, return_logits=False, num_micro_batches=None, **_):
        was_training = self.module.training
        self.module.eval()
        loss, logits = self._exec(data_iter, train=False, return_logits=return_logits,
                                  num_micro=num_micro_batches)
        self.module.train(was_training)
        if return_logits:
            out = torch.cat(logits, dim=0) if logits else None
            return loss, out
        return loss
