"""Tensor-parallel linear layers whose collective runs INSIDE the tcgen05 GEMM kernel.

The NCCL formulation of a Megatron layer (``megatron/mpu/layers.py:560-590,760-794`` and the mappings in
``megatron/mpu/mappings.py``) serialises "all-gather, then GEMM" and "GEMM, then reduce-scatter / all-reduce".
Here the GEMM kernel (``ops/csrc/comm_gemm_sm100.cu``) reads gathered operands tile by tile straight from the peers'
symmetric memory with TMA and pushes scattered outputs tile by tile into the owner's receive buffer, so NVLink
traffic overlaps the tensor-core work:

====================  =========================================  ==========================================
layer, pass           NCCL form                                  fused form
====================  =========================================  ==========================================
column, fwd (SP)      all-gather(x) ; y = x W^T                  publish(x) ; GEMM reading A from all ranks
column, dgrad (SP)    dx = dy W ; reduce-scatter                 GEMM pushing row blocks ; owner-side reduce
column, wgrad (SP)    all-gather(x) ; dW = dy^T x                publish(x) ; GEMM reading B from all ranks
row, fwd (SP)         y = x W^T ; reduce-scatter                 GEMM pushing row blocks ; reduce (+bias, +res)
row, dgrad+wgrad(SP)  all-gather(dy) ; two GEMMs                 publish(dy) ; two GEMMs reading A remotely
row, fwd (no SP)      y = x W^T ; all-reduce                     push ; reduce ; broadcast-store ; copy
column, dgrad(no SP)  dx = dy W ; all-reduce                     same
====================  =========================================  ==========================================

Buffers are double-buffered by epoch parity and guarded by "done" flags, so any interleaving of these ops that is
identical on all ranks of the group is safe.  Shapes the kernels do not take (row shard not a multiple of 128,
groups larger than 8, CPU tensors) fall back to the NCCL mappings; ``NEOX_FUSED_TP_COMM=0`` disables the fused path.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import gemm as G
from ..ops import native
from . import comms_logger, mpu
from . import symm_mem as S
from ..ops.linear import main_grad_of

_workspaces = {}
# CTAs of a broadcasting GEMM's grid that copy instead of computing (each moves roughly 40-60 GB/s)
COPY_CTAS = int(os.environ.get("NEOX_COPY_CTAS", "16"))


def fused_all_gather(world=None) -> bool:
    """Whether gathered operands arrive by the in-GEMM broadcast or by an NCCL all-gather before a plain GEMM.
    ``NEOX_FUSED_AG=1`` / ``0`` forces one; by default the broadcast is used from 4 ranks up.  Measured at h=6144,
    8192 tokens: on 2 B200s the broadcast shares the L2 ports with the GEMM's operand traffic and ends up 5-10%
    slower than "NCCL all-gather, then GEMM"; on 4 it is 2-7% faster (each rank sends the same shard to three
    peers while the NCCL ring needs three serial steps).  The pushed reduce-scatter / all-reduce is faster than
    its NCCL form at every size and is always on."""
    mode = os.environ.get("NEOX_FUSED_AG", "auto")
    if mode in ("0", "1"):
        return mode == "1"
    if world is None:
        world = mpu.get_model_parallel_world_size()
    return world >= 4


def overlap_tail() -> bool:
    """Whether the reduction tail of a data-gradient GEMM is enqueued on a side stream so that it overlaps the
    weight-gradient GEMM of the same layer (``NEOX_OVERLAP_AR_TAIL=0`` keeps everything on one stream)."""
    return os.environ.get("NEOX_OVERLAP_AR_TAIL", "1") != "0"


def _nccl_gather_rows(x2):
    ws = workspace()
    full = torch.empty(x2.shape[0] * ws.world, x2.shape[1], device=x2.device, dtype=x2.dtype)
    dist.all_gather_into_tensor(full, x2, group=ws.group)
    return full


def enabled() -> bool:
    return os.environ.get("NEOX_FUSED_TP_COMM", "1") != "0" and torch.cuda.is_available()


class _Gather:
    """Handle of one gathered tensor (see ``Workspace.begin_gather``)."""
    __slots__ = ("epoch", "shard", "rows", "cols", "buf", "full")


class Workspace:
    """Per-process-group symmetric buffers + epoch counters."""

    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.pad = S.SignalPad(group)
        self.bufs = {"ag": [None, None], "recv": [None, None], "gath": [None, None], "full": [None, None]}
        self.cnt = None
        self._send_cnt = None
        self._views = {}
        self.ag_epoch = 0
        self.bc_epoch = 0
        self.rs_epoch = 0
        self._gath_last = [0, 0]

    side = None     # stream of deferred reduction tails

    def _buf(self, kind, parity, nbytes):
        b = self.bufs[kind][parity]
        if b is None or b.nbytes < nbytes:
            # collective growth: shapes are identical on all ranks, so every rank gets here at the same op
            if b is not None:
                self._views = {k: v for k, v in self._views.items() if k[0] != id(b)}
                b.close()
            size = (int(nbytes * 1.0) + (1 << 21) - 1) // (1 << 21) * (1 << 21)
            b = S.SymmBuffer(size, self.group)
            self.bufs[kind][parity] = b
        return b

    # ------------------------------------------------------------------ all-gather side
    def publish(self, x2):
        """Stage this rank's shard ``x2`` ([rows, cols] bf16, contiguous) for a stand-alone ``gather``."""
        assert x2.is_contiguous() and x2.dtype == torch.bfloat16
        self.ag_epoch += 1
        e = self.ag_epoch
        nbytes = x2.numel() * 2
        buf = self._buf("ag", e & 1, nbytes)
        L = native.lib()
        rc = L.neox_symm_publish(native.ptr(x2), ctypes.c_void_p(buf.local), None, ctypes.c_ulonglong(nbytes),
                                 self.pad.word(S.AG_DONE), ctypes.c_uint((e - 2) & 0xFFFFFFFF), self.pad.c_ptrs,
                                 self.world, self.rank, S.AG_READY, ctypes.c_uint(e), self.pad.word(S.CTR_PUBLISH),
                                 ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_symm_publish")
        return e

    def all_gather(self, x2):
        """Stand-alone all-gather along dim 0 by peer loads (no GEMM to hide it behind)."""
        e = self.publish(x2)
        return self.gather(e, x2.shape[0], x2.shape[1])

    def begin_gather(self, x2):
        """Open a gathered view of the row-sharded tensor whose local shard is ``x2`` ([rows, cols] bf16).

        Returns a handle ``h``; ``h.full`` is a [rows * world, cols] tensor over this rank's symmetric gathered
        buffer.  Its contents arrive while a ``gemm(..., gather=h, bcast=True)`` runs on every rank of the group
        (each rank broadcasts its own shard); a GEMM given ``dep="a"`` / ``"b"`` may read ``h.full`` as that operand
        and waits block by block.  ``h.full`` may be read by any later kernel once such a dependent GEMM has finished,
        until ``release(h)``; a tensor that must outlive that has to be cloned.
        """
        assert x2.is_contiguous() and x2.dtype == torch.bfloat16 and x2.shape[0] % 128 == 0
        comms_logger.record_fused("fused_all_gather_gemm", x2.numel() * 2 * self.world, self.world)
        self.bc_epoch += 1
        e = self.bc_epoch
        rows, cols = x2.shape
        assert rows * self.world // 128 <= S.CNT_WORDS
        F = self._buf("full", e & 1, rows * self.world * cols * 2)
        if self.cnt is None:
            self.cnt = S.SymmBuffer(2 * S.CNT_WORDS * 4, self.group)
        h = _Gather()
        h.epoch, h.shard, h.rows, h.cols, h.buf = e, x2, rows, cols, F
        # building a tensor over foreign memory costs ~1 ms of host time: keep one view per buffer and shape
        key = (id(F), rows, cols)
        view = self._views.get(key)
        if view is None:
            view = F.tensor((rows * self.world, cols))
            self._views[key] = view
        h.full = view
        return h

    def release(self, h):
        """All local reads of ``h.full`` have been launched: let the peers overwrite the buffer (two epochs on)."""
        par = h.epoch & 1
        rc = native.lib().neox_symm_release(ctypes.c_void_p(self.cnt.local + par * S.CNT_WORDS * 4),
                                            int(self.world * h.rows // 128), self.pad.c_ptrs, self.world, self.rank,
                                            S.BC_DONE, ctypes.c_uint(h.epoch & 0xFFFFFFFF),
                                            ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_symm_release")
        h.full = None

    def gemm(self, a, b, a_mn=False, b_mn=False, out=None, out_dtype=torch.bfloat16, bias=None, add=None,
             act=G.ACT_NONE, want_preact=False, gather=None, bcast=False, dep=None, scatter=None):
        """The tcgen05 GEMM with an optional broadcast job and an optional pushed output.

        ``gather``: handle from ``begin_gather``.  ``bcast``: this kernel sends the local shard to every rank's
        gathered buffer while it computes.  ``dep`` ("a" / "b" / None): that operand is ``gather.full``; its loads
        wait for the blocks to arrive.  ``scatter = (recv, epoch)``: push the output row blocks to their owners
        instead of writing ``out``.
        """
        if a_mn:
            K, M = a.shape
        else:
            M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        pre = None
        if scatter is None:
            if out is None:
                out = torch.empty(M, N, device=a.device, dtype=out_dtype)
            if want_preact:
                pre = torch.empty(M, N, device=a.device, dtype=torch.bfloat16)
        if gather is not None:
            h = gather
            par = h.epoch & 1
            cnt_off = par * S.CNT_WORDS * 4
            if self._send_cnt is None:
                self._send_cnt = torch.zeros(S.CNT_WORDS, device=a.device, dtype=torch.int32)
            g_args = (native.ptr(h.shard) if bcast else None, h.buf.c_ptrs, self.cnt.offset_ptrs(cnt_off),
                      native.ptr(self._send_cnt), self.pad.word(S.BC_DONE), ctypes.c_uint((h.epoch - 2) & 0xFFFFFFFF), int(h.rows),
                      ctypes.c_longlong(h.cols * 2), ctypes.c_void_p(self.cnt.local + cnt_off), int(dep == "a"),
                      int(dep == "b"))
        else:
            assert not bcast and dep is None
            g_args = (None, None, None, None, None, ctypes.c_uint(0), 0, ctypes.c_longlong(0), None, 0, 0)
        if scatter is not None:
            recv, e = scatter
            sc_args = (1, int(M // self.world), recv.c_ptrs, self.pad.word(S.RS_DONE),
                       ctypes.c_uint((e - 2) & 0xFFFFFFFF))
            sig = (S.RS_READY, ctypes.c_uint(e & 0xFFFFFFFF))
        else:
            sc_args = (0, 0, None, None, ctypes.c_uint(0))
            sig = (-1, ctypes.c_uint(0))
        L = native.lib()
        rc = L.neox_comm_gemm(
            native.ptr(a), native.ptr(b), native.ptr(out), M, N, K, ctypes.c_longlong(a.stride(0)),
            ctypes.c_longlong(b.stride(0)), ctypes.c_longlong(out.stride(0) if out is not None else N), int(a_mn),
            int(b_mn), int(out is not None and out.dtype == torch.float32), native.ptr(bias), native.ptr(add),
            ctypes.c_longlong(add.stride(0) if add is not None else 0),
            int(add is not None and add.dtype == torch.float32), native.ptr(pre),
            ctypes.c_longlong(pre.stride(0) if pre is not None else 0), int(act), self.world, self.rank,
            *g_args, *sc_args, self.pad.c_ptrs, sig[0], sig[1], -1, ctypes.c_uint(0), self.pad.word(S.CTR_GEMM),
            int(COPY_CTAS), ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_comm_gemm")
        return (out, pre) if want_preact else out

    def gather(self, epoch, rows, cols, last_reader=True):
        """Materialise the concatenation of the published [rows, cols] shards as a local tensor."""
        out = torch.empty(rows * self.world, cols, device=torch.device("cuda", torch.cuda.current_device()),
                          dtype=torch.bfloat16)
        buf = self.bufs["ag"][epoch & 1]
        rc = native.lib().neox_symm_gather(buf.c_ptrs, native.ptr(out), ctypes.c_ulonglong(rows * cols * 2),
                                           self.pad.word(S.AG_READY), ctypes.c_uint(epoch & 0xFFFFFFFF),
                                           self.pad.c_ptrs, self.world, self.rank,
                                           S.AG_DONE if last_reader else -1, self.pad.word(S.CTR_GCOPY),
                                           ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_symm_gather")
        return out

    def gemm_reduce(self, a, b, b_mn, bias=None, residual=None, all_reduce=False, partial_bias=None,
                    partial_add=None, gather=None, defer=False):
        """``reduce_over_ranks(a @ op(b) + partial_bias + partial_add) + bias + residual``: returns this rank's
        [M / world, N] row block (reduce-scatter) or the whole [M, N] result (``all_reduce``).  The ``partial_*``
        terms are added to this rank's product before the reduction (in the GEMM epilogue), ``bias`` / ``residual``
        once after it (``residual`` has the shape of the result).  ``gather``: a handle whose broadcast rides on this
        GEMM as a prefetch for a later op (see ``gemm``).

        ``defer``: the reduction tail (reduce the received partial tiles, hand the result to the peers) is enqueued
        on a side stream and ``(out, join)`` is returned; work launched on the calling stream before ``join()`` --
        the weight-gradient GEMM of the same layer -- then runs while the tail waits for the peers and moves data.
        ``out`` must not be read before ``join()``."""
        M, K = a.shape
        N = b.shape[1] if b_mn else b.shape[0]
        rows = M // self.world
        comms_logger.record_fused("fused_gemm_all_reduce" if all_reduce else "fused_gemm_reduce_scatter",
                                  M * N * 2, self.world)
        self.rs_epoch += 1
        e = self.rs_epoch
        recv = self._buf("recv", e & 1, M * N * 2)
        gath = self._buf("gath", e & 1, M * N * 2) if all_reduce else None
        self.gemm(a, b, False, b_mn, bias=partial_bias, add=partial_add, gather=gather, bcast=gather is not None,
                  scatter=(recv, e))
        L = native.lib()
        out = torch.empty(M if all_reduce else rows, N, device=a.device, dtype=torch.bfloat16)
        if residual is not None:
            assert residual.is_contiguous() and residual.dtype == torch.bfloat16
        if defer:
            main = torch.cuda.current_stream()
            if self.side is None:
                self.side = torch.cuda.Stream()
            self.side.wait_stream(main)
            with torch.cuda.stream(self.side):
                self._reduce_tail(recv, gath, out, bias, residual, all_reduce, rows, M, N, e)
            side = self.side
            return out, lambda: torch.cuda.current_stream().wait_stream(side)
        self._reduce_tail(recv, gath, out, bias, residual, all_reduce, rows, M, N, e)
        return out

    def _reduce_tail(self, recv, gath, out, bias, residual, all_reduce, rows, M, N, e):
        L = native.lib()
        res_ptr = native.ptr(residual)
        if all_reduce and residual is not None:
            # the owner adds the residual rows it owns
            res_ptr = ctypes.c_void_p(residual.data_ptr() + self.rank * rows * N * 2)
        rc = L.neox_rs_reduce(ctypes.c_void_p(recv.local), native.ptr(out) if not all_reduce else None,
                              native.ptr(bias), res_ptr, self.world, self.rank, rows, N, self.pad.word(S.RS_READY),
                              ctypes.c_uint(e), self.pad.c_ptrs, S.RS_DONE, self.pad.word(S.CTR_REDUCE),
                              gath.c_ptrs if all_reduce else None, self.pad.word(S.AR_DONE),
                              ctypes.c_uint(self._gath_last[e & 1]), S.AR_READY,
                              ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_rs_reduce")
        if all_reduce:
            self._gath_last[e & 1] = e
            rc = L.neox_gathered_copy(ctypes.c_void_p(gath.local), native.ptr(out), ctypes.c_ulonglong(M * N * 2),
                                      self.pad.word(S.AR_READY), ctypes.c_uint(e), self.pad.c_ptrs, self.world,
                                      self.rank, S.AR_DONE, self.pad.word(S.CTR_GCOPY),
                                      ctypes.c_void_p(native.stream_ptr()))
            native.check(rc, "neox_gathered_copy")


def workspace(group=None) -> Workspace:
    group = group if group is not None else mpu.get_model_parallel_group()
    key = id(group)
    ws = _workspaces.get(key)
    if ws is None:
        ws = Workspace(group)
        _workspaces[key] = ws
    return ws


def reset():
    """Drop all workspaces (collective).  Call before destroying the process groups."""
    for ws in _workspaces.values():
        for pair in ws.bufs.values():
            for b in pair:
                if b is not None:
                    b.close()
        if ws.cnt is not None:
            ws.cnt.close()
        ws.pad.close()
    _workspaces.clear()


def eligible(x2, weight, world, sharded_rows=None) -> bool:
    """Shapes / dtypes the fused kernels accept.  ``sharded_rows``: rows of the per-rank row block."""
    if not enabled() or world < 2 or world > S.MAX_RANKS:
        return False
    if not (x2.is_cuda and x2.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and weight.is_contiguous()):
        return False
    if sharded_rows is None or sharded_rows % 128 or sharded_rows == 0:
        return False
    return x2.shape[-1] % 8 == 0 and weight.shape[0] % 8 == 0 and weight.shape[1] % 8 == 0


def _accumulate_wgrad(weight, fn):
    """Run the weight-gradient GEMM ``fn(out, add)``: into ``weight.main_grad`` when the engine provides it."""
    mg = main_grad_of(weight)
    if mg is not None:
        fn(mg, mg)
        weight.grad_in_main = True
        from ..ops.linear import notify_grad_ready
        notify_grad_ready(weight)
        return None
    return fn(None, None)


class _ColumnSP(torch.autograd.Function):
    """Column-parallel linear under sequence parallelism: input [rows, K] is this rank's sequence shard."""

    @staticmethod
    def forward(ctx, x, weight, bias, act, split_pre=False):
        ctx.set_materialize_grads(False)    # no zero tensor for the non-differentiable pre-activation output
        ws = workspace()
        N, K = weight.shape
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        rows = x2.shape[0]
        need_pre = act == "gelu" and any(ctx.needs_input_grad[:3])
        ctx.split_pre = split_pre
        act_id = G.ACT_GELU if act == "gelu" else G.ACT_NONE
        if fused_all_gather():
            h = ws.begin_gather(x2)
            r = ws.gemm(h.full, weight, bias=bias, act=act_id, want_preact=need_pre, gather=h, bcast=True, dep="a")
            ws.release(h)
        else:
            r = G.gemm(_nccl_gather_rows(x2), weight, bias=bias, act=act_id, want_preact=need_pre)
        out, pre = r if need_pre else (r, None)
        ctx.act, ctx.rows, ctx.x_shape, ctx.has_bias = act, rows, x.shape, bias is not None
        ctx.bias_ref = bias
        ctx.save_for_backward(x2, weight, None if split_pre else pre)
        out = out.reshape(x.shape[0] * ws.world, *x.shape[1:-1], N)
        if split_pre:
            if pre is not None:
                pre = pre.reshape(out.shape)
                ctx.mark_non_differentiable(pre)
            return out, pre
        return out

    @staticmethod
    def backward(ctx, g, g_pre=None):
        if g is None:
            return None, None, None, None, None
        ws = workspace()
        x2, weight, pre = ctx.saved_tensors
        N, K = weight.shape
        g2 = g.reshape(-1, N)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        if ctx.act == "gelu" and not ctx.split_pre:
            from ..ops.functional import dgelu_mul
            g2 = dgelu_mul(g2, pre)
        gx = gw = gb = None
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        if fused_all_gather():
            h = ws.begin_gather(x2) if need_w else None
            if need_x:
                # the data-gradient GEMM carries the broadcast of x as a prefetch for the weight-gradient GEMM
                gx = ws.gemm_reduce(g2, weight, True, gather=h).reshape(ctx.x_shape)
            if need_w:
                gw = _accumulate_wgrad(weight, lambda out, add: ws.gemm(g2, h.full, True, True, out=out, add=add,
                                                                        gather=h, bcast=not need_x, dep="b"))
                ws.release(h)
        else:
            join = None
            if need_x:
                if overlap_tail() and need_w:
                    gx, join = ws.gemm_reduce(g2, weight, True, defer=True)
                    gx = gx.reshape(ctx.x_shape)
                else:
                    gx = ws.gemm_reduce(g2, weight, True).reshape(ctx.x_shape)
            if need_w:
                full = _nccl_gather_rows(x2)
                gw = _accumulate_wgrad(weight, lambda out, add: G.gemm(g2, full, a_mn=True, b_mn=True, out=out,
                                                                       add=add))
            if join is not None:
                join()
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = OF.bias_grad(g2, ctx.bias_ref)
        return gx, gw, gb, None, None


class _Row(torch.autograd.Function):
    """Row-parallel linear with its reduction: ``reduce(x W^T [+ bias] [+ partial_add]) [+ bias] + residual``.

    ``sp``: the reduction is a reduce-scatter along dim 0 (sequence parallelism) and ``residual`` / the result are
    this rank's sequence shard; otherwise an all-reduce.  ``bias_partial`` selects whether the bias is added to this
    rank's partial product (every rank then contributes its own bias) or once after the reduction.
    """

    @staticmethod
    def forward(ctx, x, weight, bias, residual, partial_add, sp, bias_partial, dgelu_aux=None):
        ws = workspace()
        N, K = weight.shape
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        res2 = residual.reshape(-1, N).contiguous() if residual is not None else None
        add2 = partial_add.reshape(-1, N) if partial_add is not None else None
        if add2 is not None and not add2.is_contiguous():
            add2 = add2.contiguous()
        from ..ops.linear import output_is_dead
        if output_is_dead():
            # recomputation of a block's last layer: nobody reads this result (every rank takes this branch, so the
            # buffer epochs stay in step)
            out = torch.empty(x2.shape[0] // ws.world if sp else x2.shape[0], N, dtype=x2.dtype, device=x2.device)
        else:
            out = ws.gemm_reduce(x2, weight, False, bias=None if bias_partial else bias, residual=res2,
                                 all_reduce=not sp, partial_bias=bias if bias_partial else None, partial_add=add2)
        ctx.x_shape, ctx.sp, ctx.bias_partial = x.shape, sp, bias_partial
        ctx.has_bias, ctx.has_res, ctx.has_add = bias is not None, residual is not None, partial_add is not None
        ctx.bias_ref = bias
        ctx.add_shape = partial_add.shape if partial_add is not None else None
        ctx.save_for_backward(x2, weight, dgelu_aux.reshape(-1, K) if dgelu_aux is not None else None)
        lead = x.shape[0] // ws.world if sp else x.shape[0]
        return out.reshape(lead, *x.shape[1:-1], N)

    @staticmethod
    def backward(ctx, g):
        ws = workspace()
        x2, weight, aux2 = ctx.saved_tensors
        N, K = weight.shape
        g2 = g.reshape(-1, N)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        gx = gw = gb = g_add = None

        def dgrad(gf):
            # the GeLU' factor of the producing layer rides in this GEMM's epilogue
            if aux2 is not None:
                return G.gemm(gf, weight, a_mn=False, b_mn=True, act=G.ACT_DGELU, aux=aux2)
            return G.gemm(gf, weight, a_mn=False, b_mn=True)

        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_add = ctx.has_add and ctx.needs_input_grad[4]
        need_full_bias = ctx.has_bias and ctx.bias_partial and ctx.needs_input_grad[2]
        if not ctx.sp:
            g_full = g2                                   # backward of an all-reduce is the identity
            if need_x:
                gx = dgrad(g_full).reshape(ctx.x_shape)
            if need_w:
                gw = _accumulate_wgrad(weight, lambda out, add: G.gemm(g_full, x2, a_mn=True, b_mn=True, out=out,
                                                                       add=add))
        else:
            # backward of the reduce-scatter is an all-gather of g: it arrives while the first GEMM that reads it runs
            if not fused_all_gather():
                g_full = _nccl_gather_rows(g2)
                if need_x:
                    gx = dgrad(g_full).reshape(ctx.x_shape)
                if need_w:
                    gw = _accumulate_wgrad(weight, lambda out, add: G.gemm(g_full, x2, a_mn=True, b_mn=True, out=out,
                                                                           add=add))
            elif need_x or need_w:
                h = ws.begin_gather(g2)
                if need_x:
                    gx = ws.gemm(h.full, weight, False, True, gather=h, bcast=True, dep="a")
                    if aux2 is not None:
                        from ..ops.functional import dgelu_mul
                        gx = dgelu_mul(gx, aux2)
                    gx = gx.reshape(ctx.x_shape)
                if need_w:
                    gw = _accumulate_wgrad(weight, lambda out, add: ws.gemm(h.full, x2, True, True, out=out, add=add,
                                                                            gather=h, bcast=not need_x, dep="a"))
                g_full = h.full.clone() if (need_add or need_full_bias) else None
                ws.release(h)
            else:
                g_full = ws.all_gather(g2)
        if need_add:
            g_add = g_full.reshape(ctx.add_shape)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            # post-reduction bias under SP: partial over this rank's shard, summed with the other replicated grads
            gb = OF.bias_grad(g_full if (ctx.bias_partial or not ctx.sp) else g2, ctx.bias_ref)
        return gx, gw, gb, (g if ctx.has_res else None), g_add, None, None, None


class _ColumnAR(torch.autograd.Function):
    """Column-parallel linear without sequence parallelism: forward is local, the data gradient is all-reduced."""

    @staticmethod
    def forward(ctx, x, weight, bias, act, split_pre=False):
        ctx.set_materialize_grads(False)    # no zero tensor for the non-differentiable pre-activation output
        N, K = weight.shape
        x2 = x.reshape(-1, K)
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        need_pre = act == "gelu" and any(ctx.needs_input_grad[:3])
        r = G.gemm(x2, weight, bias=bias, act=G.ACT_GELU if act == "gelu" else G.ACT_NONE, want_preact=need_pre)
        out, pre = r if need_pre else (r, None)
        ctx.act, ctx.x_shape, ctx.has_bias, ctx.split_pre = act, x.shape, bias is not None, split_pre
        ctx.bias_ref = bias
        ctx.save_for_backward(x2, weight, None if split_pre else pre)
        out = out.reshape(*x.shape[:-1], N)
        if split_pre:
            if pre is not None:
                pre = pre.reshape(out.shape)
                ctx.mark_non_differentiable(pre)
            return out, pre
        return out

    @staticmethod
    def backward(ctx, g, g_pre=None):
        if g is None:
            return None, None, None, None, None
        ws = workspace()
        x2, weight, pre = ctx.saved_tensors
        N, K = weight.shape
        g2 = g.reshape(-1, N)
        if not g2.is_contiguous():
            g2 = g2.contiguous()
        if ctx.act == "gelu" and not ctx.split_pre:
            from ..ops.functional import dgelu_mul
            g2 = dgelu_mul(g2, pre)
        gx = gw = gb = None
        join = None
        if ctx.needs_input_grad[0]:
            # the all-reduce tail of the data gradient runs beside the weight-gradient GEMM
            if overlap_tail() and ctx.needs_input_grad[1]:
                gx, join = ws.gemm_reduce(g2, weight, True, all_reduce=True, defer=True)
                gx = gx.reshape(ctx.x_shape)
            else:
                gx = ws.gemm_reduce(g2, weight, True, all_reduce=True).reshape(ctx.x_shape)
        if ctx.needs_input_grad[1]:
            gw = _accumulate_wgrad(weight, lambda out, add: G.gemm(g2, x2, a_mn=True, b_mn=True, out=out, add=add))
        if join is not None:
            join()
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = OF.bias_grad(g2, ctx.bias_ref)
        return gx, gw, gb, None, None


def column_linear(x, weight, bias, act, sequence_parallel, split_pre=False):
    return (_ColumnSP if sequence_parallel else _ColumnAR).apply(x, weight, bias, act, split_pre)


def row_linear(x, weight, bias, residual, sequence_parallel, partial_add=None, bias_partial=False, dgelu_aux=None):
    return _Row.apply(x, weight, bias, residual, partial_add, bool(sequence_parallel), bool(bias_partial), dgelu_aux)
