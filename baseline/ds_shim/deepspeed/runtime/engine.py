"""Stand-in training engine: mixed-precision optimizer wrapper + gradient accumulation + data-parallel reduction.

Follows what DeepSpeed does for the configurations the reference ships:
  * bf16: parameters cast to bf16 and flattened per optimizer group; gradients of every micro-batch are added into an
    fp32 flat buffer; at the accumulation boundary the buffer is averaged over the data-parallel group (NCCL), the
    global gradient norm is taken with tensor-parallel awareness (replicated parameters counted once), gradients
    are clipped, the wrapped optimizer updates this rank's fp32 master partition (ZeRO-1), and the updated bf16
    partition is all-gathered.
  * fp16: the same with dynamic loss scaling and overflow skipping.
"""
import torch
import torch.distributed as dist

from .bf16_optimizer import BF16_Optimizer


class _Group:
    __slots__ = ("lp", "lp_flat", "hp_grad", "grad_views", "master", "shard", "numel", "counted")


def _flatten_into(params, pad_to, dtype, device):
    n = sum(p.numel() for p in params)
    total = (n + pad_to - 1) // pad_to * pad_to
    flat = torch.zeros(total, dtype=dtype, device=device)
    return flat, n


class MixedPrecisionOptimizer:
    """Wraps the optimizer the reference built; holds fp32 master partitions and fp32 gradient accumulators."""

    def __init__(self, inner, dtype, dp_group, norm_groups, tp_rank, clip, fp16_cfg=None):
        self.optimizer = inner
        self.dtype = dtype
        self.dp_group = dp_group
        self.dp_world = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
        self.norm_groups = [g for g in norm_groups if g is not None and dist.get_world_size(g) > 1]
        self.clip = float(clip or 0.0)
        self.overflow = False
        self.fp16 = dtype == torch.float16
        fp16_cfg = fp16_cfg or {}
        self.dynamic = self.fp16 and float(fp16_cfg.get("loss_scale", 0)) == 0
        self.cur_scale = 1.0
        if self.fp16:
            self.cur_scale = float(2 ** fp16_cfg.get("initial_scale_power", 16)) if self.dynamic \
                else float(fp16_cfg["loss_scale"])
        self.scale_window = int(fp16_cfg.get("loss_scale_window", 1000))
        self.min_scale = float(fp16_cfg.get("min_loss_scale", 1))
        self.hysteresis = self.cur_hysteresis = int(fp16_cfg.get("hysteresis", 2))
        self.good_steps = 0
        self._global_norm = None
        self.groups = []
        for pg in inner.param_groups:
            lp = [p for p in pg["params"]]
            g = _Group()
            g.lp = lp
            if not lp:
                g.numel = 0
                self.groups.append(g)
                continue
            dev = lp[0].device
            g.lp_flat, g.numel = _flatten_into(lp, self.dp_world * 8, dtype, dev)
            off = 0
            for p in lp:
                n = p.numel()
                g.lp_flat[off:off + n].copy_(p.data.reshape(-1))
                p.data = g.lp_flat[off:off + n].view_as(p.data)
                off += n
            g.hp_grad = torch.zeros(g.lp_flat.numel(), dtype=torch.float32, device=dev)
            g.grad_views, off = [], 0
            for p in lp:
                g.grad_views.append(g.hp_grad[off:off + p.numel()].view_as(p))
                off += p.numel()
            g.shard = g.lp_flat.numel() // self.dp_world
            lo = self.dp_rank * g.shard
            g.master = torch.nn.Parameter(g.lp_flat[lo:lo + g.shard].float())
            g.master.grad = g.hp_grad[lo:lo + g.shard]
            # parameters replicated over tensor-parallel ranks count once in the gradient norm
            g.counted = torch.tensor([1.0 if (getattr(p, "model_parallel", False) or tp_rank == 0) and
                                      not getattr(p, "ds_pipe_replicated", False) else 0.0 for p in lp],
                                     dtype=torch.float32, device=dev)
            pg["params"] = [g.master]
            self.groups.append(g)
        inner.state.clear()

    @property
    def param_groups(self):
        return self.optimizer.param_groups

    @property
    def state(self):
        return self.optimizer.state

    def state_dict(self):
        return {"optimizer_state_dict": self.optimizer.state_dict(), "cur_scale": self.cur_scale}

    def load_state_dict(self, sd):
        self.optimizer.load_state_dict(sd["optimizer_state_dict"])
        self.cur_scale = sd.get("cur_scale", self.cur_scale)

    def zero_grad(self, set_to_none=True):
        for g in self.groups:
            for p in g.lp:
                p.grad = None

    def accumulate(self):
        """Add this micro-batch's low-precision gradients into the fp32 accumulators and drop them."""
        for g in self.groups:
            views, grads = [], []
            for p, v in zip(g.lp, g.grad_views):
                if p.grad is not None:
                    views.append(v)
                    grads.append(p.grad)
                    p.grad = None
            for v, gr in zip(views, grads):
                v.add_(gr)

    def step(self):
        live = [g for g in self.groups if g.numel]
        if self.dp_world > 1:
            for g in live:
                dist.all_reduce(g.hp_grad, op=dist.ReduceOp.AVG, group=self.dp_group)
        sq = None
        for g in live:
            norms = torch.stack(torch._foreach_norm(g.grad_views))
            s = (norms.double() ** 2 * g.counted.double()).sum()
            sq = s if sq is None else sq + s
        for grp in self.norm_groups:
            dist.all_reduce(sq, group=grp)
        norm = sq.sqrt().float() / self.cur_scale
        self._global_norm = norm
        if self.fp16:
            self.overflow = not bool(torch.isfinite(norm))
            if self.overflow:
                if self.dynamic:
                    self.cur_hysteresis -= 1
                    if self.cur_hysteresis <= 0:
                        self.cur_scale = max(self.cur_scale / 2, self.min_scale)
                    self.good_steps = 0
                for g in live:
                    g.hp_grad.zero_()
                return False
        coef = torch.full_like(norm, 1.0 / self.cur_scale)
        if self.clip > 0:
            coef = coef * torch.clamp(self.clip / (norm + 1e-6), max=1.0)
        for g in live:
            g.master.grad.mul_(coef)
        self.optimizer.step()
        for g in live:
            lo = self.dp_rank * g.shard
            g.lp_flat[lo:lo + g.shard].copy_(g.master.data)
            if self.dp_world > 1:
                dist.all_gather_into_tensor(g.lp_flat, g.lp_flat[lo:lo + g.shard].clone(), group=self.dp_group)
            g.hp_grad.zero_()
        if self.dynamic:
            self.good_steps += 1
            self.cur_hysteresis = self.hysteresis
            if self.good_steps % self.scale_window == 0:
                self.cur_scale *= 2
        return True


class BF16MixedPrecisionOptimizer(MixedPrecisionOptimizer, BF16_Optimizer):
    pass


def precision_of(cfg):
    if (cfg.get("bf16") or {}).get("enabled") or (cfg.get("bfloat16") or {}).get("enabled"):
        return torch.bfloat16
    if (cfg.get("fp16") or {}).get("enabled"):
        return torch.float16
    return torch.float32


def wrap_optimizer(inner, cfg, dtype, dp_group, norm_groups, tp_rank):
    cls = BF16MixedPrecisionOptimizer if dtype == torch.bfloat16 else MixedPrecisionOptimizer
    return cls(inner, dtype, dp_group, norm_groups, tp_rank, cfg.get("gradient_clipping", 0.0), cfg.get("fp16"))


class ShimEngine(torch.nn.Module):
    def __init__(self, model, optimizer, lr_scheduler, cfg, mpu, model_parameters=None):
        super().__init__()
        if optimizer is None:
            raise RuntimeError("the deepspeed stand-in needs the client optimizer (config-built optimizers are not provided)")
        self.cfg = cfg
        self.mpu = mpu
        self.dtype = precision_of(cfg)
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
        self.device = dev
        model.to(dev)
        if self.dtype != torch.float32:
            model.to(self.dtype)
        self.module = model
        dp_group = mpu.get_data_parallel_group() if mpu is not None else None
        mp_group = mpu.get_model_parallel_group() if mpu is not None else None
        tp_rank = mpu.get_model_parallel_rank() if mpu is not None else 0
        self.dp_world = dist.get_world_size(dp_group) if dist.is_initialized() else 1
        self.optimizer = wrap_optimizer(optimizer, cfg, self.dtype, dp_group if dist.is_initialized() else None,
                                        [mp_group], tp_rank)
        self.lr_scheduler = lr_scheduler
        self._gas = int(cfg.get("gradient_accumulation_steps", 1) or 1)
        self._mbs = int(cfg.get("train_micro_batch_size_per_gpu", 1) or 1)
        self.micro_steps = 0
        self.global_steps = 0
        self.global_samples = 0
        self.skipped_steps = 0
        self.has_moe_layers = False

    def forward(self, *a, **k):
        return self.module(*a, **k)

    def gradient_accumulation_steps(self):
        return self._gas

    def train_micro_batch_size_per_gpu(self):
        return self._mbs

    def train_batch_size(self):
        return self._mbs * self._gas * self.dp_world

    def zero_optimization_stage(self):
        return int((self.cfg.get("zero_optimization") or {}).get("stage", 0))

    def is_gradient_accumulation_boundary(self):
        return (self.micro_steps + 1) % self._gas == 0

    def get_global_grad_norm(self):
        n = self.optimizer._global_norm
        return None if n is None else float(n)

    def backward(self, loss, **_):
        scaled = loss.float() * (self.optimizer.cur_scale / self._gas)
        scaled.backward()
        self.optimizer.accumulate()
        return loss

    def step(self, **_):
        if self.is_gradient_accumulation_boundary():
            ok = self.optimizer.step()
            if ok and self.lr_scheduler is not None:
                self.lr_scheduler.step()
            if not ok:
                self.skipped_steps += 1
            self.global_steps += 1
            self.global_samples += self.train_batch_size()
        self.micro_steps += 1

    def save_checkpoint(self, *a, **k):
        raise RuntimeError("checkpoint writing is not provided by the deepspeed stand-in")

    def load_checkpoint(self, *a, **k):
        raise RuntimeError("checkpoint loading is not provided by the deepspeed stand-in")
