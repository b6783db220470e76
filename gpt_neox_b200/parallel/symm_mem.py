"""Symmetric (peer-mapped) device memory for the ranks of one NVLink/NVSwitch domain.

A ``SymmBuffer`` is the same-sized device allocation on every rank of a process group, with every rank
holding a mapped pointer to every other rank's copy (CUDA IPC handles exchanged through the group).
Kernels address a peer's copy with ordinary loads / stores / non-multicast TMA loads over NVLink.

``SignalPad`` is a small symmetric buffer of 32-bit epoch flags.  A producer publishes ``flag[me] = epoch`` in
every consumer's pad with a system-scope release store after a system fence; consumers poll THEIR OWN pad (local
memory) with acquire loads, bounded in time.  Epochs only grow, so flags are never reset and a late reader can never
miss an event.

The reference has no counterpart: it reaches peers only through NCCL (``megatron/mpu/mappings.py``).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import native

MAX_RANKS = 8

# word offsets inside the signal pad (each block has one slot per rank)
AG_READY, AG_DONE, RS_READY, RS_DONE, AR_READY, AR_DONE = 0, 8, 16, 24, 32, 40
CTR_PUBLISH, CTR_GEMM, CTR_REDUCE, CTR_GCOPY = 48, 49, 50, 51
BC_DONE = 56                      # gathered-buffer release flags of the in-GEMM broadcast
CNT_WORDS = 4096                  # block counters per buffer parity
PAD_BYTES = 4096


def _ull_array(vals):
    arr = (ctypes.c_ulonglong * MAX_RANKS)()
    for i, v in enumerate(vals):
        arr[i] = v
    return arr


class SymmBuffer:
    """``nbytes`` of device memory on every rank of ``group``; ``ptrs[r]`` is rank r's copy as seen from here."""

    def __init__(self, nbytes: int, group=None):
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert self.world <= MAX_RANKS, "symmetric memory spans at most one 8-GPU NVLink domain"
        self.nbytes = int(nbytes)
        L = native.lib()
        p = ctypes.c_void_p()
        native.check(L.neox_symm_alloc(ctypes.byref(p), ctypes.c_ulonglong(self.nbytes)), "neox_symm_alloc")
        self.local = p.value
        handle = (ctypes.c_ubyte * 64)()
        native.check(L.neox_ipc_get_handle(ctypes.c_void_p(self.local), handle), "neox_ipc_get_handle")
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle), group=group)
        self.ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                self.ptrs.append(self.local)
                continue
            buf = (ctypes.c_ubyte * 64).from_buffer_copy(h)
            q = ctypes.c_void_p()
            native.check(L.neox_ipc_open(buf, ctypes.byref(q)), "neox_ipc_open")
            self.ptrs.append(q.value)
        self.c_ptrs = _ull_array(self.ptrs)
        # every rank has mapped every copy before anyone writes through a mapping
        dist.barrier(group=group)

    def offset_ptrs(self, byte_offset: int):
        return _ull_array([p + byte_offset for p in self.ptrs])

    def close(self):
        """Collective: unmaps the peers' copies and frees the local one."""
        if self.local is None:
            return
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        L = native.lib()
        for r, p in enumerate(self.ptrs):
            if r != self.rank:
                L.neox_ipc_close(ctypes.c_void_p(p))
        dist.barrier(group=self.group)
        L.neox_symm_free(ctypes.c_void_p(self.local))
        self.local = None
        self.ptrs = []

    def tensor(self, shape, dtype=torch.bfloat16, byte_offset=0, rank=None):
        """A torch view of (part of) one copy; for tests and debugging (the kernels take raw pointers)."""
        ptr = self.ptrs[self.rank if rank is None else rank] + byte_offset
        typestr = {torch.bfloat16: "<u2", torch.float16: "<f2", torch.float32: "<f4", torch.int32: "<i4",
                   torch.uint8: "|u1"}[dtype]

        class _Iface:
            __cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3}

        t = torch.as_tensor(_Iface(), device=torch.device("cuda", torch.cuda.current_device()))
        return t.view(dtype) if dtype == torch.bfloat16 else t


class SignalPad(SymmBuffer):
    def __init__(self, group=None):
        super().__init__(PAD_BYTES, group)

    def word(self, index: int):
        """Address of word ``index`` of the LOCAL pad."""
        return ctypes.c_void_p(self.local + 4 * index)
