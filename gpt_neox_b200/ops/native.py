"""ctypes binding of ``libneox_b200.so`` (CUDA kernels) and ``libneox_host.so`` (host C++).

The kernels expose a plain C ABI (raw device pointers + a stream handle), so no PyTorch headers are
needed at build time and a rebuild takes seconds.  ``lib()`` raises if the CUDA library cannot be
loaded: on a machine with a GPU a missing extension is an error, never a silent eager fallback.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIBDIR = Path(__file__).resolve().parent / "_lib"
_cuda_lib = None
_host_lib = None

c_void_p, c_int, c_ll, c_float = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float

ERRORS = {1: "alignment", 2: "tensor-map encode", 3: "driver/alloc", 4: "launch", 5: "shape", 6: "too large"}


class NativeError(RuntimeError):
    pass


def _load(name: str, builder: str):
    path = _LIBDIR / name
    if not path.exists() and os.environ.get("NEOX_B200_NO_AUTOBUILD", "0") != "1":
        from . import build
        getattr(build, builder)()
    if not path.exists():
        raise NativeError(f"{path} is missing; run `python -m gpt_neox_b200.ops.build`")
    return ctypes.CDLL(str(path))


launch_count = 0   # number of kernel-launching library calls made by this process (see bench.py)


class _CountingLib:
    """Proxy over the CDLL that counts calls into kernel launchers (``neox_*`` entry points that take a
    stream); pure queries such as ``neox_read_status`` are not counted."""
    _NOT_LAUNCHES = {"neox_read_status", "neox_norm_bwd_blocks", "neox_sm_count_c"}

    def __init__(self, cdll):
        self._cdll = cdll
        self._cache = {}

    def __getattr__(self, name):
        fn = self._cache.get(name)
        if fn is None:
            raw = getattr(self._cdll, name)
            if name in self._NOT_LAUNCHES:
                fn = raw
            else:
                def fn(*args, _raw=raw):
                    global launch_count
                    launch_count += 1
                    return _raw(*args)
            self._cache[name] = fn
        return fn

    def has(self, name):
        return hasattr(self._cdll, name)


def lib():
    """The CUDA kernel library (loaded once)."""
    global _cuda_lib
    if _cuda_lib is None:
        _cuda_lib = _CountingLib(_load("libneox_b200.so", "build_cuda"))
    return _cuda_lib


def host_lib():
    """The host-only C++ helper library (loaded once)."""
    global _host_lib
    if _host_lib is None:
        _host_lib = _load("libneox_host.so", "build_host")
    return _host_lib


def available() -> bool:
    """True when kernels can run: a CUDA device is visible (the library itself must then load)."""
    return torch.cuda.is_available()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def check(rc: int, what: str):
    if rc != 0:
        raise NativeError(f"{what} failed: {ERRORS.get(rc, rc)}")


def read_status() -> int:
    """Synchronise and return (then clear) the device status word; non-zero = a bounded wait expired."""
    return int(lib().neox_read_status())
