"""Mixture-of-experts MLP block with expert parallelism.

Capabilities of the two MoE back-ends the reference can be configured with
(``megatron/model/transformer.py:1076-1164``): DeepSpeed-style top-k gating with a capacity factor
(token dropping, ``moe_min_capacity``) and MegaBlocks-style dropless routing (``moe_token_dropping:
false``), optional GLU experts (``moe_glu``), router jitter, fp32 load-balancing statistics, and expert
parallelism over ``moe_expert_parallel_size`` ranks of the data-parallel group.

Data flow for T local tokens, E experts, top-k::

    probs = softmax(router(x))                       [T, E]
    (w, e) = topk(probs)                             [T, k]      (weights renormalised when k > 1)
    sort the T*k assignments by expert -> contiguous per-expert segments (capacity applied here)
    all-to-all over the expert-parallel group: every rank receives the segments of ITS experts
    per local expert: h = act(seg W1^T) W2^T         tcgen05 GEMMs on the variable-length segments
    all-to-all back, un-sort, y[token] += w * out

The auxiliary load-balancing loss returned with the output is ``E * sum_e f_e * P_e`` (``f_e`` fraction of
assignments routed to expert e, ``P_e`` mean router probability); ``training.py`` scales it by
``moe_loss_coeff``.  Expert weights are tagged ``expert_parallel`` so the optimizer reduces their gradients
over the expert-data-parallel group only.
"""
from __future__ import annotations

import math
import os

import torch
import torch.distributed as dist
import torch.nn as nn
import torch.nn.functional as F

from ..ops import functional as OF
from ..ops import gemm as G
from ..ops import moe_ops as MO
from ..ops.linear import linear as fused_linear
from ..parallel import mappings as M
from ..parallel import moe_comm, mpu
from ..ops.linear import main_grad_of


class _AllToAll(torch.autograd.Function):
    """Variable-split all-to-all over the expert-parallel group; backward swaps the split lists."""

    @staticmethod
    def forward(ctx, x, out_splits, in_splits, group):
        ctx.group, ctx.out_splits, ctx.in_splits = group, out_splits, in_splits
        out = x.new_empty((sum(out_splits), *x.shape[1:]))
        dist.all_to_all_single(out, x.contiguous(), output_split_sizes=out_splits, input_split_sizes=in_splits,
                               group=group)
        return out

    @staticmethod
    def backward(ctx, g):
        out = g.new_empty((sum(ctx.in_splits), *g.shape[1:]))
        dist.all_to_all_single(out, g.contiguous(), output_split_sizes=ctx.in_splits,
                               input_split_sizes=ctx.out_splits, group=ctx.group)
        return out, None, None, None


class _ExpertOutCombine(torch.autograd.Function):
    """Output projection of all local experts fused with the return all-to-all.

    forward: for expert e, ``hdn[a:b] @ w2[e]^T`` is computed by the tcgen05 GEMM whose epilogue stores row i at
    ``dest[i]`` -- the slot of that token in the combine buffer of the rank it came from (peer memory).  A flag tells
    every rank when this rank's rows are in place; the rows arriving here are then copied out.
    backward: the gradient rows travel the opposite way (peer push), are put back into expert-major order and feed
    the two gradient GEMMs of every expert (weight gradients accumulate into ``w2.main_grad`` when present).
    """

    @staticmethod
    def forward(ctx, hdn, w2, bounds, perm_t, perm, src, block_start, back, matrix, grp):
        import numpy as np
        comm = moe_comm.comm_for(grp)
        h = w2.shape[1]
        row_bytes = h * 2
        e, recv_off = comm.begin_push(back)
        buf = comm.push_buffer(e, back, row_bytes)
        base = np.asarray(buf.ptrs, dtype=np.int64)
        roff = np.asarray(recv_off, dtype=np.int64)
        dest = base[src] + (roff[src] + perm - np.asarray(block_start, dtype=np.int64)[src]) * row_bytes
        dest_t = torch.from_numpy(dest).to(hdn.device, non_blocking=True)
        for ei, (a, b) in enumerate(bounds):
            if b > a:
                G.gemm_rowmap(hdn[a:b], w2[ei], dest_t[a:b])
        ys = comm.finish_push(e, buf, back, h, hdn.device)
        ctx.save_for_backward(hdn, w2, perm_t)
        ctx.bounds, ctx.matrix, ctx.grp = bounds, matrix, grp
        return ys

    @staticmethod
    def backward(ctx, g):
        hdn, w2, perm_t = ctx.saved_tensors
        g_src = moe_comm.comm_for(ctx.grp).exchange(g.contiguous(), ctx.matrix)      # back on the expert rank
        g_e = g_src.index_select(0, perm_t)
        d_hdn = torch.empty_like(hdn)
        mg = main_grad_of(w2)
        gw = None if mg is not None else torch.zeros_like(w2)
        for ei, (a, b) in enumerate(ctx.bounds):
            if b <= a:
                continue
            G.gemm(g_e[a:b], w2[ei], a_mn=False, b_mn=True, out=d_hdn[a:b])
            if mg is not None:
                G.gemm(g_e[a:b], hdn[a:b], a_mn=True, b_mn=True, out=mg[ei], add=mg[ei])
            else:
                G.gemm(g_e[a:b], hdn[a:b], a_mn=True, b_mn=True, out=gw[ei])
        if mg is not None:
            w2.grad_in_main = True
            from ..ops.linear import notify_grad_ready
            notify_grad_ready(w2)
        return d_hdn, gw, None, None, None, None, None, None, None, None


class Router(nn.Module):
    def __init__(self, neox_args, num_experts):
        super().__init__()
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        self.layer = nn.Linear(neox_args.hidden_size, num_experts, bias=False, device=dev,
                               dtype=neox_args.params_dtype)
        nn.init.normal_(self.layer.weight, mean=0.0, std=neox_args.init_method_std)
        self.top_k = neox_args.moe_top_k
        self.jitter_eps = neox_args.moe_jitter_eps
        self.fp32 = neox_args.moe_lbl_in_fp32

    def forward(self, x):
        if self.training and self.jitter_eps:
            noise = torch.empty_like(x).uniform_(1.0 - self.jitter_eps, 1.0 + self.jitter_eps)
            x = x * noise
        logits = self.layer(x)
        # router probabilities always in fp32 (``moe_lbl_in_fp32`` only matters for the statistics built from them);
        # softmax, top-k, renormalisation and the expert histogram are one kernel on a GPU
        return MO.router(logits, self.top_k)


class ParallelMoE(nn.Module):
    def __init__(self, neox_args, init_method, output_layer_init_method, num_experts):
        super().__init__()
        self.num_experts = num_experts
        self.ep = mpu.get_expert_parallel_world_size()
        assert num_experts % self.ep == 0, f"{num_experts} experts not divisible by expert-parallel size {self.ep}"
        self.local_experts = num_experts // self.ep
        self.top_k = neox_args.moe_top_k
        self.token_dropping = neox_args.moe_token_dropping
        self.train_cf = neox_args.moe_train_capacity_factor
        self.eval_cf = neox_args.moe_eval_capacity_factor
        self.min_capacity = neox_args.moe_min_capacity
        self.glu = neox_args.moe_glu
        self.activation = neox_args.activation
        h = neox_args.hidden_size
        ffn_full = neox_args.intermediate_size or int((neox_args.expansion_factor or 4) * h)
        # expert tensor parallelism (``enable_expert_tensor_parallelism``): every expert's hidden dimension is split
        # over the tensor-parallel group (first projection column-parallel, second row-parallel, one all-reduce of
        # the combined output); without it every tensor-parallel rank holds whole experts
        tp = mpu.get_model_parallel_world_size()
        self.expert_tp = bool(neox_args.enable_expert_tensor_parallelism) and tp > 1
        if self.expert_tp:
            assert ffn_full % tp == 0, f"expert hidden size {ffn_full} not divisible by tensor-parallel size {tp}"
        tp_rank = mpu.get_model_parallel_rank() if self.expert_tp else 0
        ffn = ffn_full // tp if self.expert_tp else ffn_full
        self.ffn = ffn
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        dt = neox_args.params_dtype
        self.router = Router(neox_args, num_experts)
        n_in = ffn * (2 if self.glu else 1)
        self.w1 = nn.Parameter(torch.empty(self.local_experts, n_in, h, device=dev, dtype=dt))
        self.w2 = nn.Parameter(torch.empty(self.local_experts, h, ffn, device=dev, dtype=dt))
        # Every expert is initialised from its own seed (a function of the GLOBAL expert id) at full size and then
        # sliced, so the weights depend neither on how experts are spread over expert-parallel ranks nor on the
        # tensor-parallel degree.
        ep_rank = mpu.get_expert_parallel_rank()
        lo, hi = tp_rank * ffn, (tp_rank + 1) * ffn
        for e in range(self.local_experts):
            gid = ep_rank * self.local_experts + e
            with torch.random.fork_rng(devices=[]):
                torch.manual_seed(neox_args.seed + 7919 * (gid + 1))
                tmp1 = torch.empty(ffn_full * (2 if self.glu else 1), h, dtype=torch.float)
                tmp2 = torch.empty(h, ffn_full, dtype=torch.float)
                init_method(tmp1)
                output_layer_init_method(tmp2)
            if self.glu:      # [gate; up] halves are sharded separately
                tmp1 = torch.cat([tmp1[lo:hi], tmp1[ffn_full + lo:ffn_full + hi]])
            else:
                tmp1 = tmp1[lo:hi]
            with torch.no_grad():
                self.w1[e].copy_(tmp1)
                self.w2[e].copy_(tmp2[:, lo:hi])
        if self.expert_tp:
            self.w1.model_parallel, self.w1.partition_dim, self.w1.partition_stride = True, 1, 2 if self.glu else 1
            self.w2.model_parallel, self.w2.partition_dim, self.w2.partition_stride = True, 2, 1
        if self.ep > 1:
            self.w1.expert_parallel = True
            self.w2.expert_parallel = True
        self.w1.moe_expert = self.w2.moe_expert = True
        # None: grouped expert GEMMs whenever the kernels take the shapes (GPU); True forces the grouped data flow
        # through its eager statement (CPU oracle), False keeps the per-expert loop
        self.grouped = None

    # ------------------------------------------------------------------ expert compute
    def _expert(self, e, seg):
        if seg.shape[0] == 0:
            return seg.new_zeros((0, self.w2.shape[1]))
        w1, w2 = self.w1[e], self.w2[e]
        if self.glu:
            hdn = OF.gated_act(fused_linear(seg, w1), "swiglu" if self.activation in ("swiglu", "silu") else "geglu")
        elif self.activation == "gelu":
            hdn = fused_linear(seg, w1, act="gelu")
        else:
            hdn = OF.get_activation(self.activation)(fused_linear(seg, w1))
        return fused_linear(hdn, w2)

    def _hidden(self, e, seg):
        """First half of expert ``e``: projection + activation."""
        w1 = self.w1[e]
        if self.glu:
            return OF.gated_act(fused_linear(seg, w1), "swiglu" if self.activation in ("swiglu", "silu") else "geglu")
        if self.activation == "gelu":
            return fused_linear(seg, w1, act="gelu")
        return OF.get_activation(self.activation)(fused_linear(seg, w1))

    def _experts_fused_combine(self, xr, pieces, matrix, out_splits, grp):
        """Expert MLPs whose output projection writes every row straight into the combine buffer of the rank the
        token came from (per-row destination table in the GEMM epilogue): the return all-to-all is part of the GEMM."""
        import numpy as np
        L = self.local_experts
        # expert-major order of the received rows, and for every row its source rank and position in that block
        block_start = np.concatenate(([0], np.cumsum(out_splits)))[:-1]
        perm, src, bounds, lo = [], [], [], 0
        for e in range(L):
            n_e = 0
            for o, n, r in pieces[e]:
                if n:
                    perm.append(np.arange(o, o + n, dtype=np.int64))
                    src.append(np.full(n, r, dtype=np.int64))
                    n_e += n
            bounds.append((lo, lo + n_e))
            lo += n_e
        perm = np.concatenate(perm) if perm else np.zeros(0, dtype=np.int64)
        src = np.concatenate(src) if src else np.zeros(0, dtype=np.int64)
        perm_t = torch.from_numpy(perm).to(xr.device, non_blocking=True)
        xe = xr.index_select(0, perm_t)
        hdn = torch.cat([self._hidden(e, xe[a:b]) for e, (a, b) in enumerate(bounds) if b > a])
        back = [list(c) for c in zip(*matrix)]          # rows this rank returns to rank r = rows r sent here
        return _ExpertOutCombine.apply(hdn, self.w2, bounds, perm_t, perm, src, block_start, back, matrix, grp)

    def _activate(self, x_pad, counts):
        """First expert projection + activation over the padded expert-major matrix."""
        if self.glu:
            kind = "swiglu" if self.activation in ("swiglu", "silu") else "geglu"
            return OF.gated_act(MO.grouped_linear(x_pad, self.w1, counts), kind)
        if self.activation == "gelu":
            return MO.grouped_linear(x_pad, self.w1, counts, act="gelu")
        return OF.get_activation(self.activation)(MO.grouped_linear(x_pad, self.w1, counts))

    def _use_grouped(self, x):
        if self.grouped is not None:
            return self.grouped
        mode = os.environ.get("NEOX_MOE_GROUPED", "auto")
        if mode == "0":                                         # per-expert loop
            return False
        if mode != "1" and x.shape[1] > 2048:
            # experts this large fill the machine one at a time and run on the CTA-pair GEMM, which is 12-16 % faster
            # than the one-CTA kernel the grouped modes use (measured at hidden 4096, expert hidden 14336)
            return False
        probe = x.new_empty(128, x.shape[1])
        return MO.grouped_kernel_ok(probe, self.w1) and MO.grouped_kernel_ok(x.new_empty(128, self.ffn), self.w2)

    def _forward_grouped(self, x, w, idx, counts):
        """All local experts in two grouped GEMM launches; no value is read back by the host."""
        T, k = idx.shape
        cap = self._capacity(T) if self.token_dropping else None
        row_of, kept = MO.plan_rows(idx, counts, cap)
        xs = MO.dispatch(x, row_of, MO.padded_rows(T * k, self.num_experts))
        out = MO.grouped_linear(self._activate(xs, kept), self.w2, kept)
        return MO.combine(out, row_of, w)

    def _experts_grouped(self, xr, recv_l):
        """Local experts over the rows received from the expert-parallel group (ordered by source rank, then local
        expert): re-ordered into the padded expert-major matrix, two grouped GEMM launches, and back."""
        import numpy as np
        L = self.local_experts
        n_e = [sum(recv_l[r][e] for r in range(self.ep)) for e in range(L)]
        start, row = [], 0
        for n in n_e:
            start.append(row)
            row += (n + MO.PAD - 1) // MO.PAD * MO.PAD
        rows = max(128, (row + 127) // 128 * 128)
        dst, fill = [], [0] * L
        for r in range(self.ep):
            for e in range(L):
                n = recv_l[r][e]
                dst.append(np.arange(start[e] + fill[e], start[e] + fill[e] + n, dtype=np.int64))
                fill[e] += n
        dst_t = torch.from_numpy(np.concatenate(dst)).to(xr.device, non_blocking=True)
        counts = torch.tensor(n_e, dtype=torch.int64).to(xr.device, non_blocking=True)
        xe = torch.zeros(rows, xr.shape[1], dtype=xr.dtype, device=xr.device).index_copy(0, dst_t, xr)
        out = MO.grouped_linear(self._activate(xe, counts), self.w2, counts)
        return out.index_select(0, dst_t)

    def _capacity(self, tokens):
        cf = self.train_cf if self.training else self.eval_cf
        return max(self.min_capacity, int(math.ceil(cf * tokens * self.top_k / self.num_experts)))

    def forward(self, hidden_states):
        y, lbl = self._forward(hidden_states)
        if self.expert_tp:
            y = M.reduce_from_model_parallel_region(y)
        return y, lbl

    def _forward(self, hidden_states):
        shape = hidden_states.shape
        x = hidden_states.reshape(-1, shape[-1])
        T, E, k = x.shape[0], self.num_experts, self.top_k
        probs, w, idx, counts = self.router(x)
        if self.expert_tp:
            # the router runs replicated on the unsplit input; what enters the sharded experts is marked so that the
            # partial gradients of the expert input and of the gates are summed over the tensor-parallel group
            x = M.copy_to_model_parallel_region(x)
            w = M.copy_to_model_parallel_region(w)
        # ---- load-balancing statistics
        flat_e = idx.reshape(-1)
        f = counts.float() / float(T * k)
        P = probs.mean(dim=0)
        lbl = E * torch.sum(f.detach() * P)
        if self.ep == 1 and self._use_grouped(x):
            y = self._forward_grouped(x, w, idx, counts)
            return y.reshape(shape), lbl.to(hidden_states.dtype)
        # ---- sort assignments by expert (stable: token order preserved inside an expert)
        order = torch.argsort(flat_e, stable=True)
        sorted_e = flat_e[order]
        token_of = order // k
        keep = torch.ones_like(sorted_e, dtype=torch.bool)
        if self.token_dropping:
            cap = self._capacity(T)
            starts = torch.cumsum(counts, 0) - counts
            pos = torch.arange(T * k, device=x.device) - starts[sorted_e]
            keep = pos < cap
            counts = torch.clamp(counts, max=cap)
        sel = order[keep]
        tok = token_of[keep]
        xs = x[tok]                                              # [A, h] grouped by expert
        gate = w.reshape(-1)[sel].to(x.dtype)
        if self.ep > 1:
            grp = mpu.get_expert_parallel_group()
            send = counts.view(self.ep, self.local_experts)
            # every rank learns the whole count table in one small all-gather: [src rank, dst rank, local expert]
            table = torch.empty((self.ep, self.ep, self.local_experts), dtype=send.dtype, device=send.device)
            dist.all_gather_into_tensor(table.view(-1), send.contiguous().view(-1), group=grp)
            table_l = table.tolist()
            me = mpu.get_expert_parallel_rank()
            recv_l = [table_l[r][me] for r in range(self.ep)]
            in_splits = [sum(table_l[me][d]) for d in range(self.ep)]
            out_splits = [sum(recv_l[r]) for r in range(self.ep)]
            peer = moe_comm.eligible(xs, grp)
            if peer:
                matrix = [[sum(table_l[r][d]) for d in range(self.ep)] for r in range(self.ep)]
                xr = moe_comm.all_to_all_rows(xs, matrix, grp)
            else:
                xr = _AllToAll.apply(xs, out_splits, in_splits, grp)
            # received layout: for each source rank, its segments for local experts 0..L-1
            pieces, off = [[] for _ in range(self.local_experts)], 0
            for r in range(self.ep):
                for e in range(self.local_experts):
                    n = recv_l[r][e]
                    pieces[e].append((off, n, r))
                    off += n
            if peer and moe_comm.fused_combine_enabled() and xr.shape[0] > 0:
                ys = self._experts_fused_combine(xr, pieces, matrix, out_splits, grp)
            elif xr.shape[0] > 0 and self._use_grouped(x):
                outs = self._experts_grouped(xr, recv_l)
                if peer:
                    ys = moe_comm.all_to_all_rows(outs, [list(c) for c in zip(*matrix)], grp)
                else:
                    ys = _AllToAll.apply(outs, in_splits, out_splits, grp)
            else:
                res_parts = {}
                for e in range(self.local_experts):
                    seg = torch.cat([xr[o:o + n] for o, n, _ in pieces[e]]) if pieces[e] else xr[:0]
                    out_e = self._expert(e, seg)
                    o2 = 0
                    for o, n, _ in pieces[e]:
                        if n:                  # an empty piece shares its offset with the piece that follows it
                            res_parts[o] = out_e[o2:o2 + n]
                        o2 += n
                outs = torch.cat([res_parts[o] for o in sorted(res_parts)]) if res_parts else xr
                if peer:
                    ys = moe_comm.all_to_all_rows(outs, [list(c) for c in zip(*matrix)], grp)
                else:
                    ys = _AllToAll.apply(outs, in_splits, out_splits, grp)
        else:
            cl = counts.tolist()
            parts, off = [], 0
            for e in range(E):
                parts.append(self._expert(e, xs[off:off + cl[e]]))
                off += cl[e]
            ys = torch.cat(parts) if parts else xs
        y = torch.zeros_like(x)
        y.index_add_(0, tok, ys * gate[:, None])
        return y.reshape(shape), lbl.to(hidden_states.dtype)


class ResidualMoE(nn.Module):
    """Residual mixture of experts (DeepSpeed's ``use_residual``, which the reference passes as ``moe_use_residual``
    when ``moe_type`` is ``deepspeed``, ``megatron/model/transformer.py:1084-1100``): a dense MLP runs beside the
    experts and a learned per-token two-way softmax mixes the two outputs."""

    def __init__(self, neox_args, init_method, output_layer_init_method, num_experts, dense_mlp):
        super().__init__()
        self.moe = ParallelMoE(neox_args, init_method, output_layer_init_method, num_experts)
        self.mlp = dense_mlp
        dev = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else None
        self.coefficient = nn.Linear(neox_args.hidden_size, 2, device=dev, dtype=neox_args.params_dtype)

    def forward(self, hidden_states):
        out, lbl = self.moe(hidden_states)
        dense, bias = self.mlp(hidden_states)
        if bias is not None:
            dense = dense + bias
        coef = F.softmax(self.coefficient(hidden_states).float(), dim=-1).to(out.dtype)
        return out * coef[..., 0:1] + dense * coef[..., 1:], lbl
