"""Communication logger: counts, sizes, device time and bandwidth of every collective a run issues.

The reference hands its ``comms_logger`` block (``enabled / verbose / prof_all / prof_ops / debug``,
``megatron/neox_arguments/deepspeed_args.py:238``; switched on in ``configs/19M.yml:89-94``) to DeepSpeed, which wraps
its own communication layer and prints a table per op and message size.  This build has no such layer between the
model and ``torch.distributed``, so the logger wraps the ``torch.distributed`` entry points themselves (module
attributes, so every ``dist.all_reduce(...)`` call site is covered) and offers ``record()`` to the fused
compute+collective kernels, whose traffic never passes through ``torch.distributed``.

Timing is done with CUDA events on the calling stream and resolved lazily when the summary is printed, so logging
does not add a synchronisation per collective; an asynchronous collective is timed up to the return of its
``wait()``.  On CPU (gloo) the host clock is used.
"""
from __future__ import annotations

import functools
import time
from collections import defaultdict

import torch
import torch.distributed as dist

# op name -> (position or keyword of the payload tensor, bus-bandwidth factor as a function of the group size)
_OPS = {
    "all_reduce": ("tensor", 0, lambda n: 2.0 * (n - 1) / n),
    "broadcast": ("tensor", 0, lambda n: 1.0),
    "reduce": ("tensor", 0, lambda n: 1.0),
    "all_gather_into_tensor": ("output_tensor", 0, lambda n: (n - 1) / n),
    "reduce_scatter_tensor": ("input", 1, lambda n: (n - 1) / n),
    "all_to_all_single": ("output", 0, lambda n: (n - 1) / n),
    "all_gather": ("tensor", 1, lambda n: (n - 1) / n),
    "reduce_scatter": ("output", 0, lambda n: (n - 1) / n),
    "send": ("tensor", 0, lambda n: 1.0),
    "recv": ("tensor", 0, lambda n: 1.0),
    "isend": ("tensor", 0, lambda n: 1.0),
    "irecv": ("tensor", 0, lambda n: 1.0),
    "barrier": (None, None, lambda n: 0.0),
}
_SCALE_BY_WORLD = {"all_gather", "reduce_scatter"}   # payload argument is one rank's share


class _TimedWork:
    """Stands in for the work handle of an asynchronous collective; closes the timing record in ``wait()``."""

    def __init__(self, work, closer):
        self._work, self._closer = work, closer

    def wait(self, *a, **k):
        r = self._work.wait(*a, **k)
        if self._closer is not None:
            self._closer()
            self._closer = None
        return r

    def __getattr__(self, name):
        return getattr(self._work, name)


class CommsLogger:
    def __init__(self, enabled=False, verbose=False, prof_all=True, prof_ops=None, debug=False):
        self.enabled, self.verbose, self.prof_all, self.debug = bool(enabled), bool(verbose), bool(prof_all), bool(debug)
        self.prof_ops = list(prof_ops or [])
        # records[op][bytes] = [count, [pending (start, end) event pairs], resolved milliseconds, group size]
        self.records = defaultdict(dict)
        self._orig = {}

    # ------------------------------------------------------------------ bookkeeping
    def wants(self, op):
        return self.enabled and (self.prof_all or op in self.prof_ops)

    def _slot(self, op, nbytes, world):
        return self.records[op].setdefault(int(nbytes), [0, [], 0.0, world])

    def record(self, op, nbytes, world, ms=None, events=None):
        """One occurrence of ``op`` moving ``nbytes`` among ``world`` ranks; its duration either known (``ms``) or
        to be read later from a pair of CUDA events."""
        if not self.wants(op):
            return
        slot = self._slot(op, nbytes, world)
        slot[0] += 1
        if ms is not None:
            slot[2] += ms
        elif events is not None:
            slot[1].append(events)
        if self.verbose and (not dist.is_initialized() or dist.get_rank() == 0):
            print(f"comm op: {op} | msg size: {_fmt_bytes(nbytes)} | group size: {world}"
                  + (f" | time (ms): {ms:.3f}" if ms is not None else ""), flush=True)

    def _timer(self, op, nbytes, world, on_cuda):
        if on_cuda:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()

            def close():
                end.record()
                self.record(op, nbytes, world, events=(start, end))
        else:
            t0 = time.perf_counter()

            def close():
                self.record(op, nbytes, world, ms=(time.perf_counter() - t0) * 1e3)
        return close

    # ------------------------------------------------------------------ wrapping torch.distributed
    def _wrap(self, name):
        fn = getattr(dist, name)
        key, pos, _ = _OPS[name]

        @functools.wraps(fn)
        def logged(*args, **kwargs):
            if not self.wants(name):
                return fn(*args, **kwargs)
            payload = kwargs.get(key) if key else None
            if payload is None and pos is not None and len(args) > pos:
                payload = args[pos]
            if payload is None and name == "all_gather":
                payload = kwargs.get("tensor")
            group = kwargs.get("group")
            world = dist.get_world_size(group) if dist.is_initialized() else 1
            if name in ("send", "recv", "isend", "irecv"):
                world = 2
            nbytes = payload.numel() * payload.element_size() if torch.is_tensor(payload) else 0
            if name in _SCALE_BY_WORLD:
                nbytes *= world
            on_cuda = torch.is_tensor(payload) and payload.is_cuda
            close = self._timer(name, nbytes, world, on_cuda)
            out = fn(*args, **kwargs)
            if out is not None and hasattr(out, "wait") and (kwargs.get("async_op") or name in ("isend", "irecv")):
                return _TimedWork(out, close)
            close()
            return out

        return logged

    def install(self):
        """Replace the ``torch.distributed`` entry points by logging wrappers (idempotent)."""
        if self._orig or not self.enabled:
            return self
        for name in _OPS:
            if hasattr(dist, name):
                self._orig[name] = getattr(dist, name)
                setattr(dist, name, self._wrap(name))
        return self

    def uninstall(self):
        for name, fn in self._orig.items():
            setattr(dist, name, fn)
        self._orig = {}

    # ------------------------------------------------------------------ summary
    def _resolve(self):
        if any(slot[1] for sizes in self.records.values() for slot in sizes.values()) and torch.cuda.is_available():
            torch.cuda.synchronize()
        for sizes in self.records.values():
            for slot in sizes.values():
                for start, end in slot[1]:
                    slot[2] += start.elapsed_time(end)
                slot[1] = []

    def summary(self):
        """Rows ``(op, bytes, count, total ms, mean ms, algorithm GB/s, bus GB/s)`` sorted by op and size."""
        self._resolve()
        rows = []
        for op in sorted(self.records):
            factor = _OPS[op][2] if op in _OPS else (lambda n: 1.0)
            for nbytes in sorted(self.records[op]):
                count, _, total_ms, world = self.records[op][nbytes]
                mean = total_ms / max(count, 1)
                alg = nbytes / (mean * 1e-3) / 1e9 if mean > 0 else 0.0
                rows.append((op, nbytes, count, total_ms, mean, alg, alg * factor(max(world, 1))))
        return rows

    def log_summary(self, print_fn=print):
        rows = self.summary()
        if not rows:
            return ""
        head = f"{'Comm. Op':<28}{'Message Size':<16}{'Count':<8}{'Total Latency(ms)':<20}{'Avg Latency(ms)':<18}" \
               f"{'tput_avg (GB/s)':<18}{'busbw_avg (GB/s)':<18}"
        lines = [head]
        for op, nbytes, count, total, mean, alg, bus in rows:
            lines.append(f"{op:<28}{_fmt_bytes(nbytes):<16}{count:<8}{total:<20.2f}{mean:<18.3f}{alg:<18.2f}{bus:<18.2f}")
        text = "\n".join(lines)
        if not dist.is_initialized() or dist.get_rank() == 0:
            print_fn(text)
        return text

    def reset(self):
        self.records.clear()


def _fmt_bytes(n):
    for unit in ("B", "KB", "MB", "GB"):
        if n < 1024 or unit == "GB":
            return f"{n:.2f} {unit}" if unit != "B" else f"{int(n)} B"
        n /= 1024.0


_LOGGER = CommsLogger()


def get() -> CommsLogger:
    return _LOGGER


def configure(block) -> CommsLogger:
    """Build the process-wide logger from a ``comms_logger`` configuration block and install it when enabled."""
    global _LOGGER
    _LOGGER.uninstall()
    block = dict(block or {})
    _LOGGER = CommsLogger(enabled=block.get("enabled", False), verbose=block.get("verbose", False),
                          prof_all=block.get("prof_all", True), prof_ops=block.get("prof_ops"),
                          debug=block.get("debug", False))
    return _LOGGER.install()


def record_fused(op, nbytes, world):
    """Called by the fused compute+collective kernels' host side: the NVLink traffic of one launch (no separate
    duration -- the transfer overlaps the GEMM inside one kernel, so only count and size are meaningful)."""
    if _LOGGER.enabled:
        _LOGGER.record(op, nbytes, world, ms=0.0)
