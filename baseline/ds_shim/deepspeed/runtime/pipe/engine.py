"""Stand-in pipeline engine: 1F1B over the stages of a PipelineModule with NCCL point-to-point transfers.

`train_batch(data_iter)` runs `gradient_accumulation_steps` micro-batches through the one-forward-one-backward
schedule, then takes one optimizer step.  Stage boundaries carry every tensor the previous stage returned (the
reference passes `(hidden_states, attention_mask)`); with `set_has_attention_mask(True)` the last one carries no
gradient.  Sends and receives that can meet in the steady state are issued as one batched group.
"""
import torch
import torch.distributed as dist

from ..engine import precision_of, wrap_optimizer

_DTYPES = [torch.float32, torch.float16, torch.bfloat16, torch.int64, torch.int32, torch.bool, torch.uint8]


class _Grid:
    """Process groups derived from the topology (every rank creates every group, as NCCL requires)."""

    def __init__(self, topo):
        rank = dist.get_rank()
        self.topo = topo
        self.coord = topo.get_coord(rank)
        self.dp_group = self.tp_group = self.pp_group = None
        for ranks in topo.get_axis_comm_lists("data"):
            g = dist.new_group(ranks=ranks)
            if rank in ranks:
                self.dp_group = g
        for ranks in topo.get_axis_comm_lists("model"):
            g = dist.new_group(ranks=ranks)
            if rank in ranks:
                self.tp_group = g
        for ranks in topo.get_axis_comm_lists("pipe"):
            g = dist.new_group(ranks=ranks)
            if rank in ranks:
                self.pp_group, self.pp_ranks = g, ranks
        self.stage = self.coord.pipe
        self.stages = topo.get_dim("pipe")
        self.tp_rank = getattr(self.coord, "model", 0)

    def stage_rank(self, stage):
        return self.pp_ranks[stage]


class ShimPipelineEngine(torch.nn.Module):
    def __init__(self, model, optimizer, lr_scheduler, cfg, model_parameters=None):
        super().__init__()
        if optimizer is None:
            raise RuntimeError("the deepspeed stand-in needs the client optimizer")
        self.cfg = cfg
        self.dtype = precision_of(cfg)
        self.device = torch.device("cuda", torch.cuda.current_device())
        model.to(self.device)
        if self.dtype != torch.float32:
            model.to(self.dtype)
        self.module = model
        self.grid = _Grid(model.topology())
        self.stage_id, self.num_stages = self.grid.stage, self.grid.stages
        self._tied_groups = self._build_tied_groups()
        self.optimizer = wrap_optimizer(optimizer, cfg, self.dtype, self.grid.dp_group,
                                        [self.grid.tp_group, self.grid.pp_group], self.grid.tp_rank)
        self.lr_scheduler = lr_scheduler
        self.micro_batches = int(cfg.get("gradient_accumulation_steps", 1) or 1)
        self._mbs = int(cfg.get("train_micro_batch_size_per_gpu", 1) or 1)
        self.dp_world = dist.get_world_size(self.grid.dp_group)
        self.batch_fn = None
        self.has_attention_mask = False
        self.global_steps = 0
        self.global_samples = 0
        self.has_moe_layers = False
        self._recv_meta = None          # shapes / dtypes of what the previous stage sends
        self._sent_meta = False
        self._grad_meta = None

    # ---- API the reference uses
    def set_has_attention_mask(self, v):
        self.has_attention_mask = bool(v)

    def set_batch_fn(self, fn):
        self.batch_fn = fn

    def is_first_stage(self):
        return self.stage_id == 0

    def is_last_stage(self):
        return self.stage_id == self.num_stages - 1

    def gradient_accumulation_steps(self):
        return self.micro_batches

    def train_micro_batch_size_per_gpu(self):
        return self._mbs

    def train_batch_size(self):
        return self._mbs * self.micro_batches * self.dp_world

    def is_gradient_accumulation_boundary(self):
        return True

    # ---- tied weights
    def _build_tied_groups(self):
        out = {}
        topo = self.module.topology()
        for key, stages in sorted(self.module.tied_stage_sets().items()):
            if len(stages) < 2:
                continue
            for d in range(topo.get_dim("data")):
                for m in range(max(1, topo.get_dim("model"))):
                    ranks = [topo.get_rank(pipe=s, data=d, model=m) for s in stages]
                    g = dist.new_group(ranks=ranks)
                    if dist.get_rank() in ranks:
                        out[key] = (g, ranks)
            if key in self.module.tied_modules and self.stage_id != stages[0]:
                for p in self.module.tied_modules[key].parameters():
                    p.ds_pipe_replicated = True
        for key, (g, ranks) in out.items():       # same initial value everywhere
            w = getattr(self.module.tied_modules[key], self.module.tied_weight_attrs[key])
            dist.broadcast(w.data, src=ranks[0], group=g)
        return out

    def _reduce_tied_grads(self):
        for key, (g, _) in self._tied_groups.items():
            w = getattr(self.module.tied_modules[key], self.module.tied_weight_attrs[key])
            if w.grad is not None:
                dist.all_reduce(w.grad, group=g)

    # ---- p2p helpers
    def _send_meta(self, tensors, dst):
        head = torch.tensor([len(tensors)], dtype=torch.int64, device=self.device)
        dist.send(head, dst)
        for t in tensors:
            m = torch.tensor([t.dim(), _DTYPES.index(t.dtype)] + list(t.shape), dtype=torch.int64, device=self.device)
            dist.send(torch.tensor([m.numel()], dtype=torch.int64, device=self.device), dst)
            dist.send(m, dst)

    def _recv_meta_from(self, src):
        head = torch.zeros(1, dtype=torch.int64, device=self.device)
        dist.recv(head, src)
        metas = []
        for _ in range(int(head)):
            n = torch.zeros(1, dtype=torch.int64, device=self.device)
            dist.recv(n, src)
            m = torch.zeros(int(n), dtype=torch.int64, device=self.device)
            dist.recv(m, src)
            m = m.tolist()
            metas.append((tuple(m[2:2 + m[0]]), _DTYPES[m[1]]))
        return metas

    def _ops_send_act(self, outs):
        nxt = self.grid.stage_rank(self.stage_id + 1)
        if not self._sent_meta:
            self._send_meta(outs, nxt)
            self._sent_meta = True
        return [dist.P2POp(dist.isend, t.contiguous(), nxt) for t in outs]

    def _ops_recv_act(self):
        prv = self.grid.stage_rank(self.stage_id - 1)
        if self._recv_meta is None:
            self._recv_meta = self._recv_meta_from(prv)
        bufs = [torch.empty(s, dtype=d, device=self.device) for s, d in self._recv_meta]
        return bufs, [dist.P2POp(dist.irecv, b, prv) for b in bufs]

    def _grad_tensors(self, outs):
        k = len(outs) - 1 if (self.has_attention_mask and len(outs) > 1) else len(outs)
        return [t for t in outs[:k] if t.is_floating_point()]

    @staticmethod
    def _run(ops):
        if ops:
            for w in dist.batch_isend_irecv(ops):
                w.wait()

    # ---- one micro-batch forward / backward
    def _load(self):
        batch = next(self._data_iter) if self._data_iter is not None else None
        if self.batch_fn is not None:
            batch = self.batch_fn(batch)
        return batch

    def _forward(self, recvd):
        inputs = labels = None
        if self.is_first_stage() or self.is_last_stage():
            inputs, labels = self._load()
        if not self.is_first_stage():
            k = len(recvd) - 1 if (self.has_attention_mask and len(recvd) > 1) else len(recvd)
            for t in recvd[:k]:
                if t.is_floating_point():
                    t.requires_grad_(True)
            inputs = tuple(recvd) if len(recvd) > 1 else recvd[0]
        out = self.module(inputs)
        if self.is_last_stage():
            loss = self.module.loss_fn(out, labels)
            self._losses.append(loss.detach())
            return recvd, (loss,)
        outs = tuple(out) if isinstance(out, (tuple, list)) else (out,)
        return recvd, outs

    def _backward(self, recvd, outs, grads):
        if self.is_last_stage():
            (outs[0].float() * (self.optimizer.cur_scale / self.micro_batches)).backward()
        else:
            torch.autograd.backward(self._grad_tensors(outs), grads)
        in_grads = None
        if not self.is_first_stage():
            in_grads = [t.grad for t in self._grad_tensors(recvd)]
        return in_grads

    def _recv_grad_ops(self, outs):
        nxt = self.grid.stage_rank(self.stage_id + 1)
        bufs = [torch.empty_like(t) for t in self._grad_tensors(outs)]
        return bufs, [dist.P2POp(dist.irecv, b, nxt) for b in bufs]

    def _send_grad_ops(self, in_grads):
        prv = self.grid.stage_rank(self.stage_id - 1)
        return [dist.P2POp(dist.isend, g.contiguous(), prv) for g in in_grads]

    # ---- schedule
    def train_batch(self, data_iter=None):
        self.module.train()
        self._data_iter = data_iter
        self._losses = []
        M, first, last = self.micro_batches, self.is_first_stage(), self.is_last_stage()
        warm = min(self.num_stages - self.stage_id - 1, M)
        steady = M - warm
        queue = []

        recvd = ()
        if not first:
            recvd, ops = self._ops_recv_act()
            self._run(ops)
        for i in range(warm):
            r, outs = self._forward(recvd)
            queue.append((r, outs))
            ops = [] if last else self._ops_send_act(outs)
            nxt_recv = ()
            if not first and (i + 1 < warm or steady > 0):
                nxt_recv, rops = self._ops_recv_act()
                ops = ops + rops
            self._run(ops)
            recvd = nxt_recv
        for i in range(steady):
            r, outs = self._forward(recvd)
            queue.append((r, outs))
            grads = None
            if not last:                                   # send activation, receive its gradient's predecessor
                gb, gops = self._recv_grad_ops(queue[0][1])
                self._run(self._ops_send_act(outs) + gops)
                grads = gb
            r0, o0 = queue.pop(0)
            in_grads = self._backward(r0, o0, grads)
            self.optimizer.accumulate()
            ops = [] if first else self._send_grad_ops(in_grads)
            recvd = ()
            if not first and i + 1 < steady:
                recvd, rops = self._ops_recv_act()
                ops = ops + rops
            self._run(ops)
        while queue:
            r0, o0 = queue.pop(0)
            grads = None
            if not last:
                grads, gops = self._recv_grad_ops(o0)
                self._run(gops)
            in_grads = self._backward(r0, o0, grads)
            self.optimizer.accumulate()
            if not first:
                self._run(self._send_grad_ops(in_grads))

        # tied weights were accumulated into fp32 already; reduce there
        self._reduce_tied_hp_grads()
        ok = self.optimizer.step()
        if ok and self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.global_steps += 1
        self.global_samples += self.train_batch_size()

        # mean loss: averaged over micro-batches and data-parallel ranks on the last stage, broadcast along the pipe
        loss = torch.stack(self._losses).float().mean() if last else torch.zeros((), device=self.device)
        if last and self.dp_world > 1:
            dist.all_reduce(loss, op=dist.ReduceOp.AVG, group=self.grid.dp_group)
        dist.broadcast(loss, src=self.grid.stage_rank(self.num_stages - 1), group=self.grid.pp_group)
        return loss

    def _reduce_tied_hp_grads(self):
        if not self._tied_groups:
            return
        views = {}
        for g in self.optimizer.groups:
            for p, v in zip(g.lp, g.grad_views):
                views[id(p)] = v
        for key, (grp, _) in self._tied_groups.items():
            w = getattr(self.module.tied_modules[key], self.module.tied_weight_attrs[key])
            if id(w) in views:
                dist.all_reduce(views[id(w)], group=grp)

    def eval_batch(self, data_iter, return_logits=False, **_):
        raise RuntimeError("eval_batch is not provided by the deepspeed stand-in")
