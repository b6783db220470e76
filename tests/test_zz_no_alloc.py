"""The allocation-free LayerNorm-backward entry point, called through its exported C symbol.

It exists for callers that cannot allocate device memory when they call into the library (all memory
already reserved by their framework's allocator, or no tolerance for cudaMalloc's device-wide
synchronisation).  The regular entry point wants a caller-provided scratch buffer; this one uses a
static device array inside the library.  Both must produce the same numbers, also when the shared
scratch still holds the previous call's partial sums -- hence two calls in a row with different data.
This file sorts last on purpose: a failure here cannot hide the result of any other test.
"""
import ctypes
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

LIB = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "gpt_neox_b200", "ops", "_lib",
                   "libneox_b200.so")


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr())


def _run_both(lib, rows, cols, dtype, seed):
    code = {torch.bfloat16: 0, torch.float32: 1, torch.float16: 2}[dtype]
    torch.manual_seed(seed)
    dev = "cuda"
    x = torch.randn(rows, cols, device=dev, dtype=dtype)
    g = torch.randn(rows, cols, device=dev, dtype=dtype)
    gamma = (1 + 0.1 * torch.randn(cols, device=dev)).to(dtype)
    mean = x.float().mean(-1).contiguous()
    rstd = torch.rsqrt(x.float().var(-1, unbiased=False) + 1e-5).contiguous()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    outs = []
    for which in ("regular", "noalloc"):
        dx = torch.empty_like(x)
        dgamma = torch.empty(cols, device=dev, dtype=torch.float32)
        dbeta = torch.empty(cols, device=dev, dtype=torch.float32)
        if which == "regular":
            nblk = lib.neox_norm_bwd_blocks(rows)
            ws = torch.empty(2 * nblk * cols, device=dev, dtype=torch.float32)
            rc = lib.neox_layernorm_bwd(_ptr(g), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dx), _ptr(dgamma),
                                        _ptr(dbeta), _ptr(ws), rows, cols, code, stream)
        else:
            rc = lib.neox_layernorm_bwd_noalloc(_ptr(g), _ptr(x), _ptr(gamma), _ptr(mean), _ptr(rstd), _ptr(dx),
                                                _ptr(dgamma), _ptr(dbeta), rows, cols, code, stream)
        assert rc == 0, (which, rc, lib.neox_noalloc_last_error())
        torch.cuda.synchronize()
        outs.append((dx.float(), dgamma, dbeta))
    return outs


def test_noalloc_layernorm_backward_matches_regular_entry_point():
    lib = ctypes.CDLL(LIB)                      # the raw exported symbols, no Python wrapper in between
    lib.neox_noalloc_last_error.restype = ctypes.c_char_p
    # two calls in a row: the second one finds the first one's partial sums in the shared scratch
    for seed, (rows, cols, dtype) in enumerate([(4096, 6144, torch.bfloat16), (777, 2048, torch.float32)]):
        (dx0, dg0, db0), (dx1, dg1, db1) = _run_both(lib, rows, cols, dtype, seed)
        tol = 1e-4 if dtype == torch.float32 else 3e-2
        assert torch.allclose(dx1, dx0, atol=tol, rtol=1e-2)
        assert torch.allclose(dg1, dg0, atol=tol * rows ** 0.5, rtol=2e-2)
        assert torch.allclose(db1, db0, atol=tol * rows ** 0.5, rtol=2e-2)
    # requests beyond the built-in scratch are refused with a message, not served out of bounds
    cols = 8192 + 8
    x = torch.randn(4, cols, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(cols, device="cuda")
    rc = lib.neox_layernorm_bwd_noalloc(_ptr(x), _ptr(x), _ptr(x), _ptr(f), _ptr(f), _ptr(x), _ptr(f), _ptr(f), 4,
                                        cols, 0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    assert rc == 6
    assert b"exceeds" in lib.neox_noalloc_last_error()
