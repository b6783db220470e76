"""In-tree build of the native libraries.

Two shared objects are produced next to this file (in ``_lib/``):

* ``libneox_b200.so``  -- every ``csrc/*.cu`` kernel file, compiled by nvcc for ``sm_100a`` only;
* ``libneox_host.so``  -- every ``csrc/host/*.cpp`` file (dataset index builders, CPU Adam), g++.

Objects are rebuilt only when their source (or a header) is newer.  The role of this module is the
one ``megatron/fused_kernels/__init__.py:35-143`` and ``megatron/data/Makefile`` play in the
reference, minus the per-architecture gencode list: there is exactly one target here.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIBDIR = HERE / "_lib"
OBJDIR = LIBDIR / "obj"

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-lineinfo", "-std=c++17", "--use_fast_math",
    "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-O3", "-std=c++17", "-fPIC", "-march=x86-64-v3", "-fopenmp", "-ffp-contract=off"]


def _nvcc() -> str | None:
    cand = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if cand and os.path.exists(cand) else None


def _newest_header_mtime(dirs) -> float:
    m = 0.0
    for d in dirs:
        for ext in ("*.h", "*.cuh", "*.hpp"):
            for f in Path(d).glob(ext):
                m = max(m, f.stat().st_mtime)
    return m


def _compile(cmd, src, obj, verbose):
    if verbose:
        print(" ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"compilation of {src} failed:\n{r.stdout}\n{r.stderr}")
    return obj


def _build_lib(compiler, flags, sources, out, header_dirs, link_flags, verbose, force):
    OBJDIR.mkdir(parents=True, exist_ok=True)
    hdr_m = _newest_header_mtime(header_dirs)
    jobs, objs = [], []
    for src in sources:
        obj = OBJDIR / (src.stem + ".o")
        objs.append(obj)
        if force or not obj.exists() or obj.stat().st_mtime < max(src.stat().st_mtime, hdr_m):
            jobs.append(([compiler, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], src, obj))
    with ThreadPoolExecutor(max_workers=min(8, max(1, len(jobs)))) as ex:
        list(ex.map(lambda j: _compile(j[0], j[1], j[2], verbose), jobs))
    if jobs or not out.exists():
        cmd = [compiler, "-shared", "-o", str(out), *[str(o) for o in objs], *link_flags]
        _compile(cmd, out, out, verbose)
    return out


def build_cuda(verbose: bool = False, force: bool = False) -> Path | None:
    """Compile all CUDA kernels for sm_100a.  Returns the library path (None without nvcc)."""
    nvcc = _nvcc()
    if nvcc is None:
        return None
    sources = sorted(CSRC.glob("*.cu"))
    return _build_lib(nvcc, NVCC_FLAGS, sources, LIBDIR / "libneox_b200.so", [CSRC],
                      ["-gencode", "arch=compute_100a,code=sm_100a", "-Xcompiler", "-fPIC"], verbose, force)


def build_host(verbose: bool = False, force: bool = False) -> Path | None:
    """Compile the host-only C++ helpers (no CUDA needed)."""
    cxx = shutil.which("g++")
    if cxx is None:
        return None
    sources = sorted((CSRC / "host").glob("*.cpp"))
    if not sources:
        return None
    return _build_lib(cxx, CXX_FLAGS, sources, LIBDIR / "libneox_host.so", [CSRC, CSRC / "host"],
                      ["-fopenmp"], verbose, force)


def build_all(verbose: bool = False, force: bool = False):
    return build_cuda(verbose, force), build_host(verbose, force)


if __name__ == "__main__":
    libs = build_all(verbose="-v" in sys.argv, force="-f" in sys.argv)
    print("built:", [str(l) for l in libs if l])
