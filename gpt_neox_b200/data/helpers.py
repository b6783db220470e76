"""numpy-facing wrappers of the C++ index builders in ``ops/csrc/host/data_helpers.cpp`` plus pure
Python twins used as test oracles and as a fallback when no compiler is available."""
from __future__ import annotations

import ctypes

import numpy as np


def _lib():
    from ..ops import native
    return native.host_lib()


def build_sample_idx_py(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros([num_samples + 1, 2], dtype=np.int64)
    sample, di, off = 1, 0, 0
    while sample <= num_samples:
        remaining = seq_length + 1
        while remaining != 0:
            doc_len = int(sizes[doc_idx[di]]) - off
            remaining -= doc_len
            if remaining <= 0:
                off += remaining + doc_len - 1
                remaining = 0
            else:
                di += 1
                off = 0
        out[sample] = (di, off)
        sample += 1
    return out


def build_sample_idx(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch):
    sizes = np.ascontiguousarray(sizes, dtype=np.int32)
    doc_idx = np.ascontiguousarray(doc_idx, dtype=np.int32)
    num_samples = (num_epochs * tokens_per_epoch - 1) // seq_length
    out = np.zeros([num_samples + 1, 2], dtype=np.int64)
    try:
        lib = _lib()
    except Exception:
        return build_sample_idx_py(sizes, doc_idx, seq_length, num_epochs, tokens_per_epoch)
    fn = lib.neox_build_sample_idx
    fn.restype = ctypes.c_longlong
    rows = fn(sizes.ctypes.data_as(ctypes.c_void_p), doc_idx.ctypes.data_as(ctypes.c_void_p),
              ctypes.c_longlong(len(doc_idx)), ctypes.c_int32(seq_length), ctypes.c_int32(num_epochs),
              ctypes.c_longlong(tokens_per_epoch), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_longlong(len(out)))
    if rows != num_samples + 1:
        raise RuntimeError("build_sample_idx: document order is too short for the requested number of samples")
    return out


def build_blending_indices_py(weights, size):
    n = len(weights)
    dataset_index = np.zeros(size, dtype=np.uint8)
    dataset_sample_index = np.zeros(size, dtype=np.int64)
    taken = [0] * n
    for i in range(size):
        denom = max(float(i), 1.0)
        errs = [weights[d] * denom - taken[d] for d in range(n)]
        best = int(np.argmax(errs))
        dataset_index[i] = best
        dataset_sample_index[i] = taken[best]
        taken[best] += 1
    return dataset_index, dataset_sample_index


def build_blending_indices(weights, size):
    w = np.ascontiguousarray(weights, dtype=np.float64)
    dataset_index = np.zeros(size, dtype=np.uint8)
    dataset_sample_index = np.zeros(size, dtype=np.int64)
    try:
        lib = _lib()
    except Exception:
        return build_blending_indices_py(list(w), size)
    lib.neox_build_blending_indices(dataset_index.ctypes.data_as(ctypes.c_void_p),
                                    dataset_sample_index.ctypes.data_as(ctypes.c_void_p),
                                    w.ctypes.data_as(ctypes.c_void_p), ctypes.c_int32(len(w)),
                                    ctypes.c_longlong(size))
    return dataset_index, dataset_sample_index
