"""Expert-parallel token exchange over NVLink peer memory.

``PeerAllToAll.exchange`` is a variable-split all-to-all of rows (tokens) between the ranks of the expert-parallel
group, written as two kernels of ``ops/csrc/comm_gemm_sm100.cu`` instead of an NCCL call:

* push: every rank stores the rows destined for rank d straight into d's symmetric receive buffer, at the offset
  that rank d will find them at (all ranks know the whole count matrix), one warp per row so the stores travel as
  512-byte NVLink packets, then publishes an epoch flag in every rank's signal pad;
* wait + copy: the receiver waits -- bounded -- for all source flags, moves the rows into an ordinary tensor (the
  expert GEMMs save their input for backward, and the symmetric buffer is reused two exchanges later) and tells the
  sources the buffer is free.

The reference reaches its experts through DeepSpeed / MegaBlocks all-to-alls on NCCL
(``megatron/model/transformer.py:1076-1164``).  ``NEOX_FUSED_MOE_A2A=0`` falls back to
``torch.distributed.all_to_all_single``.
"""
from __future__ import annotations

import ctypes
import os

import torch
import torch.distributed as dist

from ..ops import native
from . import symm_mem as S

A2A_READY, A2A_DONE, CTR_PUSH, CTR_COPY = 0, 8, 48, 51
_comms = {}


def enabled() -> bool:
    return os.environ.get("NEOX_FUSED_MOE_A2A", "1") != "0" and torch.cuda.is_available()


def fused_combine_enabled() -> bool:
    """Expert output GEMMs write their rows straight into the source ranks' combine buffers (``NEOX_FUSED_MOE_COMBINE=0``
    keeps GEMM and exchange separate)."""
    return os.environ.get("NEOX_FUSED_MOE_COMBINE", "1") != "0"


def _ll_array(vals):
    arr = (ctypes.c_longlong * S.MAX_RANKS)()
    for i, v in enumerate(vals):
        arr[i] = int(v)
    return arr


class PeerAllToAll:
    def __init__(self, group):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.pad = S.SignalPad(group)
        self.recv = [None, None]
        self.epoch = 0

    def _buf(self, parity, nbytes):
        b = self.recv[parity]
        if b is None or b.nbytes < nbytes:
            if b is not None:
                b.close()
            size = (int(nbytes * 1.25) + (1 << 21) - 1) // (1 << 21) * (1 << 21)
            b = S.SymmBuffer(size, self.group)
            self.recv[parity] = b
        return b

    def exchange(self, x, matrix, transpose=False):
        """``matrix[r][d]`` = rows rank r sends to rank d (identical on all ranks; ``transpose`` swaps the roles,
        which is the backward direction).  ``x``: this rank's rows grouped by destination.  Returns the received
        rows grouped by source."""
        M = [list(col) for col in zip(*matrix)] if transpose else matrix
        me, W = self.rank, self.world
        send = [M[me][d] for d in range(W)]
        recv = [M[r][me] for r in range(W)]
        recv_off = [sum(M[r][d] for r in range(me)) for d in range(W)]     # my block inside d's buffer
        send_off = [sum(send[:d]) for d in range(W)]
        x = x.contiguous()
        assert x.dtype == torch.bfloat16 and x.shape[0] == sum(send)
        h = x.shape[1]
        row_bytes = h * 2
        self.epoch += 1
        e = self.epoch
        need = max(sum(M[r][d] for r in range(W)) for d in range(W)) * row_bytes      # same number on every rank
        buf = self._buf(e & 1, max(need, 16))
        L = native.lib()
        stream = ctypes.c_void_p(native.stream_ptr())
        rc = L.neox_a2a_push(native.ptr(x) if x.numel() else ctypes.c_void_p(buf.local), buf.c_ptrs,
                             _ll_array(send_off), _ll_array(send), _ll_array(recv_off), int(row_bytes), W, me,
                             self.pad.word(A2A_DONE), ctypes.c_uint((e - 2) & 0xFFFFFFFF), self.pad.c_ptrs, A2A_READY,
                             ctypes.c_uint(e), self.pad.word(CTR_PUSH), stream)
        native.check(rc, "neox_a2a_push")
        total = sum(recv)
        out = torch.empty(max(total, 1), h, device=x.device, dtype=x.dtype)
        rc = L.neox_gathered_copy(ctypes.c_void_p(buf.local), native.ptr(out), ctypes.c_ulonglong(total * row_bytes),
                                  self.pad.word(A2A_READY), ctypes.c_uint(e), self.pad.c_ptrs, W, me, A2A_DONE,
                                  self.pad.word(CTR_COPY), stream)
        native.check(rc, "neox_gathered_copy")
        return out[:total]


    # ---- exchange whose rows are written by GEMM epilogues instead of a copy kernel
    def begin_push(self, matrix):
        """Open an exchange with count matrix ``matrix`` (as in ``exchange``) in which the caller's own kernels store
        the rows: returns ``(epoch, buf, recv_off)`` -- row ``j`` of this rank's block for destination ``d`` belongs
        at ``buf.ptrs[d] + (recv_off[d] + j) * row_bytes``.  The call waits (on the stream) until every destination
        has released the buffer."""
        me, W = self.rank, self.world
        self.epoch += 1
        e = self.epoch
        rc = native.lib().neox_wait_flags(self.pad.word(A2A_DONE), ctypes.c_uint((e - 2) & 0xFFFFFFFF), W, me,
                                          ctypes.c_void_p(native.stream_ptr()))
        native.check(rc, "neox_wait_flags")
        recv_off = [sum(matrix[r][d] for r in range(me)) for d in range(W)]
        return e, recv_off

    def push_buffer(self, e, matrix, row_bytes):
        need = max(sum(matrix[r][d] for r in range(self.world)) for d in range(self.world)) * row_bytes
        return self._buf(e & 1, max(need, 16))

    def finish_push(self, e, buf, matrix, h, device):
        """All rows of exchange ``e`` have been stored (by kernels launched on this stream): publish, wait for the
        other ranks' rows and return them as a tensor."""
        me, W = self.rank, self.world
        L = native.lib()
        stream = ctypes.c_void_p(native.stream_ptr())
        zeros = _ll_array([0] * W)
        rc = L.neox_a2a_push(ctypes.c_void_p(buf.local), buf.c_ptrs, zeros, zeros, zeros, 16, W, me,
                             self.pad.word(A2A_DONE), ctypes.c_uint((e - 2) & 0xFFFFFFFF), self.pad.c_ptrs, A2A_READY,
                             ctypes.c_uint(e), self.pad.word(CTR_PUSH), stream)
        native.check(rc, "neox_a2a_push")
        total = sum(matrix[r][me] for r in range(W))
        out = torch.empty(max(total, 1), h, device=device, dtype=torch.bfloat16)
        rc = L.neox_gathered_copy(ctypes.c_void_p(buf.local), native.ptr(out), ctypes.c_ulonglong(total * h * 2),
                                  self.pad.word(A2A_READY), ctypes.c_uint(e), self.pad.c_ptrs, W, me, A2A_DONE,
                                  self.pad.word(CTR_COPY), stream)
        native.check(rc, "neox_gathered_copy")
        return out[:total]


def comm_for(group) -> PeerAllToAll:
    key = id(group)
    c = _comms.get(key)
    if c is None:
        c = PeerAllToAll(group)
        _comms[key] = c
    return c


def reset():
    for c in _comms.values():
        for b in c.recv:
            if b is not None:
                b.close()
        c.pad.close()
    _comms.clear()


class _PeerA2AFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, matrix, group):
        ctx.matrix, ctx.group = matrix, group
        return comm_for(group).exchange(x, matrix)

    @staticmethod
    def backward(ctx, g):
        return comm_for(ctx.group).exchange(g, ctx.matrix, transpose=True), None, None


def eligible(x, group) -> bool:
    return (enabled() and x.is_cuda and x.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[1] % 8 == 0
            and dist.get_world_size(group) <= S.MAX_RANKS and native.available())


def all_to_all_rows(x, matrix, group):
    """Differentiable row exchange; ``matrix`` as in ``PeerAllToAll.exchange`` (list of lists of python ints)."""
    return _PeerA2AFn.apply(x, matrix, group)
