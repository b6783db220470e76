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
in-register); activations are sent with ``batch_isend_irecv`` so the send of micro-batch *i* and
the receive for micro-batch *i+1* are in flight while compute proceeds on the main stream.
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

    # ------------------------------------------------------------------ mode helpers
    def train(self, mode=True):
        self.module.train(mode)
        self.training = mode
        return self

    def eval(self):
        return self.train(False)

    def __call__(self, *args, **kwargs):
        return self.module(*args, **kwargs)

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
        scaled.backward(retain_graph=retain_graph)
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
        self._pre_step_grad_sync()
        if self.store_gradients:
            self.stored_gradients = [p.main_grad.detach().clone() for b in self.optimizer.buckets for p in b.params]
        ok = self.optimizer.step(grad_divisor=float(self.gas * self.dp_world_size))
        fp8.invalidate_weight_cache()          # the fused optimizer rewrites parameters through raw pointers
        if ok:
            if self.lr_scheduler is not None:
                self.lr_scheduler.step()
        else:
            self.skipped_steps += 1
        self.global_steps += 1
        self.global_samples += self.neox_args.train_batch_size

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


# ============================================================================================== pipeline
class _P2P:
    """Adjacent-stage tensor exchange with a one-time (per direction) meta handshake."""

    def __init__(self):
        self.ranks = mpu.get_pipe_parallel_ranks()
        self.stage = mpu.get_pipe_parallel_rank()
        self.group = mpu.get_pipe_parallel_group()
        self.meta = {}

    def peer(self, delta):
        return self.ranks[self.stage + delta]

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
        dist.send(buf, dst)
        self.meta[key] = ([(tuple(t.shape), t.dtype) for t in tensors], is_tuple)

    def _recv_meta(self, src, key):
        if key in self.meta:
            return self.meta[key]
        buf = torch.zeros(64, dtype=torch.int64, device=self._device())
        dist.recv(buf, src)
        h = buf.tolist()
        n, is_tuple, pos, metas = h[0], bool(h[1]), 2, []
        for _ in range(n):
            nd, dt = h[pos], h[pos + 1]
            metas.append((tuple(h[pos + 2:pos + 2 + nd]), _DTYPES[dt]))
            pos += 8
        self.meta[key] = (metas, is_tuple)
        return self.meta[key]

    def send_ops(self, tensors, delta):
        dst = self.peer(delta)
        return [dist.P2POp(dist.isend, t.contiguous(), dst) for t in tensors]

    def recv_ops(self, metas, delta):
        src = self.peer(delta)
        bufs = [torch.empty(shape, dtype=dt, device=self._device()) for shape, dt in metas]
        return bufs, [dist.P2POp(dist.irecv, b, src) for b in bufs]

    @staticmethod
    def run(ops):
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()


class PipelineEngine(NeoXEngine):
    def __init__(self, model, optimizer, lr_scheduler, neox_args, sp_sync_params=None):
        super().__init__(model, optimizer, lr_scheduler, neox_args, sp_sync_params)
        self.is_pipe_parallel = True
        self.num_stages = mpu.get_pipe_parallel_world_size()
        self.stage_id = mpu.get_pipe_parallel_rank()
        self.micro_batches = self.gas
        self.batch_fn = None
        self.has_attention_mask = False
        self.p2p = _P2P() if self.num_stages > 1 else None
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

        def recv_fwd():
            if first:
                return None
            metas, is_tuple = p2p._recv_meta(p2p.peer(-1), "act")
            state["tuple"] = is_tuple
            bufs, ops = p2p.recv_ops(metas, -1)
            _P2P.run(ops)
            return prep(bufs)

        def send_fwd(out):
            if last:
                return
            ts, is_tuple = self._tensors_of(out)
            p2p._send_meta(ts, p2p.peer(+1), "act", is_tuple)
            _P2P.run(p2p.send_ops(ts, +1))

        def grad_metas(out):
            ts, _ = self._tensors_of(out)
            return [(tuple(t.shape), t.dtype) for t in ts if t.is_floating_point()]

        def send_fwd_recv_bwd(out):
            if last:
                return None
            ts, is_tuple = self._tensors_of(out)
            p2p._send_meta(ts, p2p.peer(+1), "act", is_tuple)
            bufs, rops = p2p.recv_ops(grad_metas(out), +1)
            _P2P.run(p2p.send_ops(ts, +1) + rops)
            return bufs

        def recv_bwd(out):
            if last:
                return None
            bufs, rops = p2p.recv_ops(grad_metas(out), +1)
            _P2P.run(rops)
            return bufs

        def in_grads(recv):
            return [b.grad if b.grad is not None else torch.zeros_like(b) for b in recv if b.is_floating_point()]

        def send_bwd(recv):
            if first:
                return
            _P2P.run(p2p.send_ops(in_grads(recv), -1))

        def send_bwd_recv_fwd(recv):
            if first:
                return None
            metas, is_tuple = p2p._recv_meta(p2p.peer(-1), "act")
            bufs, rops = p2p.recv_ops(metas, -1)
            _P2P.run(p2p.send_ops(in_grads(recv), -1) + rops)
            return prep(bufs)

        def fwd(recv):
            inputs, labels = self._load_micro_batch(data_iter)
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
                for _ in range(M):
                    recv = recv_fwd()
                    out, loss = fwd(recv)
                    send_fwd(out)
        else:
            for _ in range(warm):
                recv = recv_fwd()
                out, loss = fwd(recv)
                send_fwd(out)
                queue.append((recv, out, loss))
            remaining = M - warm
            recv = recv_fwd() if remaining > 0 else None
            for i in range(remaining):
                out, loss = fwd(recv)
                grads = send_fwd_recv_bwd(out)
                queue.append((recv, out, loss))
                r0, o0, l0 = queue.pop(0)
                if warm > 0:
                    # the gradient that just arrived belongs to the OLDEST outstanding micro-batch
                    pass
                bwd(o0, l0, grads)
                if i == remaining - 1:
                    send_bwd(r0)
                    recv = None
                else:
                    recv = send_bwd_recv_fwd(r0)
            for _ in range(warm):
                r0, o0, l0 = queue.pop(0)
                grads = recv_bwd(o0)
                bwd(o0, l0, grads)
                send_bwd(r0)

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
    def train_batch(self, data_iter=None):
        self.module.train()
        loss, _ = self._exec(data_iter, train=True)
        if hasattr(self.module, "allreduce_tied_weight_gradients"):
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
