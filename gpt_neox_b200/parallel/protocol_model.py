"""Host-side replay of the peer-memory flag protocols: a small model checker for the orderings the kernels rely on.

The fused compute+collective kernels (``ops/csrc/comm_gemm_sm100.cu``) and the ZeRO-1 peer traffic synchronise through
epoch flags in symmetric memory: a producer stores data into a peer's buffer and then raises ``flag[me] = epoch`` in
the peer's signal pad; a consumer waits for ``flag >= epoch`` before it reads; buffers are reused by epoch parity and
guarded by "done" flags.  Whether such a protocol is free of races and deadlocks does not depend on the GPU: it is a
property of the sequence of waits, stores, loads and signals that every rank issues.  This module states those
sequences as data (mirroring the epoch arithmetic of ``parallel/fused_comm.py`` and ``engine/flat_optimizer.py``),
executes them for all ranks under many random interleavings, and checks that

* every load observes exactly the value the matching store of the SAME epoch wrote (nothing stale, nothing
  overwritten early), and
* all ranks run to completion (no circular wait).

Memory is modelled as sequentially consistent (the kernels use system-scope release stores and acquire loads for the
flags, with a system fence between data and flag), so this checks the protocol logic, not the fences.  It stands in
for a device-side race detector, which cannot be run on the GPUs this was developed on.  The reference has no
counterpart: it reaches peers only through NCCL.
"""
from __future__ import annotations

import random
from collections import defaultdict


class ProtocolViolation(AssertionError):
    pass


class Actor:
    """One in-order instruction stream (a CUDA stream of one rank) executing a list of operations:

    ``("wait", slot, src, value)``       local pad: flag[slot][src] >= value
    ``("signal", dst, slot, value)``     pad of rank dst: flag[slot][me] = value
    ``("write", owner, buf, idx, tag)``  memory of rank owner: buf[idx] = tag
    ``("read", owner, buf, idx, tag)``   memory of rank owner: buf[idx] must equal tag
    ``("set", name, value)`` / ``("need", name, value)``   events between the streams of one rank (stream ordering)
    """

    def __init__(self, rank, name, ops):
        self.rank, self.name, self.ops, self.pc = rank, name, list(ops), 0

    def done(self):
        return self.pc >= len(self.ops)


class Simulator:
    def __init__(self, world):
        self.world = world
        self.flags = [defaultdict(int) for _ in range(world)]      # flags[rank][(slot, src)]
        self.mem = [dict() for _ in range(world)]                  # mem[rank][(buf, idx)]
        self.events = [defaultdict(int) for _ in range(world)]     # events[rank][name]
        self.actors = []

    def add(self, rank, name, ops):
        self.actors.append(Actor(rank, name, ops))

    def _enabled(self, a):
        op = a.ops[a.pc]
        if op[0] == "wait":
            return self.flags[a.rank][(op[1], op[2])] >= op[3]
        if op[0] == "need":
            return self.events[a.rank][op[1]] >= op[2]
        return True

    def _step(self, a):
        op = a.ops[a.pc]
        kind = op[0]
        if kind == "signal":
            _, dst, slot, value = op
            if value < self.flags[dst][(slot, a.rank)]:
                raise ProtocolViolation(f"rank {a.rank}/{a.name}: flag {slot} would go backwards")
            self.flags[dst][(slot, a.rank)] = value
        elif kind == "write":
            _, owner, buf, idx, tag = op
            self.mem[owner][(buf, idx)] = tag
        elif kind == "read":
            _, owner, buf, idx, tag = op
            seen = self.mem[owner].get((buf, idx))
            if seen != tag:
                raise ProtocolViolation(f"rank {a.rank}/{a.name}: read {buf}[{idx}] of rank {owner}: expected {tag}, "
                                        f"found {seen}")
        elif kind == "set":
            self.events[a.rank][op[1]] = max(self.events[a.rank][op[1]], op[2])
        a.pc += 1

    def run(self, seed=0, max_steps=10 ** 7):
        """Execute under a random interleaving; raises ``ProtocolViolation`` on a bad read or a deadlock."""
        rng = random.Random(seed)
        for _ in range(max_steps):
            live = [a for a in self.actors if not a.done()]
            if not live:
                return
            ready = [a for a in live if self._enabled(a)]
            if not ready:
                stuck = ", ".join(f"rank {a.rank}/{a.name} at {a.ops[a.pc]}" for a in live)
                raise ProtocolViolation(f"deadlock: {stuck}")
            # run a random burst of one ready actor: long bursts let one rank race far ahead of the others
            a = rng.choice(ready)
            for _ in range(rng.choice((1, 1, 2, 5, 50))):
                if a.done() or not self._enabled(a):
                    break
                self._step(a)
        raise ProtocolViolation("step limit reached")


# ------------------------------------------------------------------------------------------------ protocols
RS_READY, RS_DONE, AR_READY, AR_DONE = "rs_ready", "rs_done", "ar_ready", "ar_done"


def gemm_all_reduce_program(world, rank, epochs, deferred_tail=False, guard_recv=True, guard_gathered=True,
                            wait_ready=True):
    """``Workspace.gemm_reduce(all_reduce=True)`` called ``epochs`` times (``parallel/fused_comm.py``):

    GEMM (push): for every owner o: wait RS_DONE[o] >= e - 2 (o has reduced the buffer of that parity), store this
    rank's partial rows into o's receive buffer of parity e & 1; then raise RS_READY[me] = e everywhere.
    Reduce: wait RS_READY[src] >= e and AR_DONE[src] >= e - 2 for all src; load all partials; store the reduced rows
    into every rank's gathered buffer of parity e & 1; raise RS_DONE[me] = AR_READY[me] = e everywhere.
    Copy: wait AR_READY[r] >= e for all r; load the gathered buffer; raise AR_DONE[me] = e everywhere.

    ``deferred_tail``: reduce and copy run on a side stream that the main stream joins before the next GEMM (the
    weight-gradient GEMM in between touches none of this).

    ``wait_ready=False`` drops the reducer's wait for the partials (the checker must then find a stale read).  The
    two ``guard_*`` switches drop the "buffer is free again" waits: replaying shows that in THIS call sequence they are
    implied by stream order (a rank can start GEMM e + 2 only after its copy of epoch e + 1, which needed every
    owner's reduction of epoch e + 1, which follows that owner's reduction of epoch e), so they are a second line of
    defence for other call sequences, not what makes this one correct."""
    main, side = [], []
    tail = side if deferred_tail else main
    for e in range(1, epochs + 1):
        par = e & 1
        order = [(rank + d) % world for d in range(1, world)] + [rank]          # remote owners first
        for o in order:
            if guard_recv:
                main.append(("wait", RS_DONE, o, e - 2))
            main.append(("write", o, f"recv{par}", rank, ("partial", e, rank)))
        for dst in range(world):
            main.append(("signal", dst, RS_READY, e))
        if deferred_tail:
            main.append(("set", "gemm", e))
            side.append(("need", "gemm", e))
        for src in range(world):
            if wait_ready:
                tail.append(("wait", RS_READY, src, e))
            if guard_gathered:
                tail.append(("wait", AR_DONE, src, e - 2))
        for src in range(world):
            tail.append(("read", rank, f"recv{par}", src, ("partial", e, src)))
        for dst in range(world):
            tail.append(("write", dst, f"gath{par}", rank, ("reduced", e, rank)))
        for dst in range(world):
            tail.append(("signal", dst, RS_DONE, e))
            tail.append(("signal", dst, AR_READY, e))
        for r in range(world):
            tail.append(("wait", AR_READY, r, e))
        for r in range(world):
            tail.append(("read", rank, f"gath{par}", r, ("reduced", e, r)))
        for dst in range(world):
            tail.append(("signal", dst, AR_DONE, e))
        if deferred_tail:
            side.append(("set", "tail", e))
            main.append(("need", "tail", e))          # join before the result is used / the next GEMM starts
    return {"main": main, "side": side} if deferred_tail else {"main": main}


READY, DONE, GATHERED = "z_ready", "z_done", "z_gathered"


def zero_peer_program(world, rank, steps, wait_done_before_zero=True):
    """One bucket of the ZeRO-1 peer traffic (``engine/flat_optimizer.py``, ``NEOX_ZERO_PEER=1``) over ``steps``
    optimizer steps, main stream and communication stream of one rank:

    main: read all parameter shards (forward / backward), write all gradient shards, hand over to the communication
    stream; after the reduction: Adam on the own shard; wait DONE[r] >= e for all r, zero the gradients; before the
    next step's first read wait GATHERED[r] >= e.
    comm: raise READY[me] = e; wait READY[r] >= e; load the own shard from every rank's gradient buffer, store the
    sum; raise DONE[me] = e; after Adam: store the updated shard into every rank's parameter buffer, raise
    GATHERED[me] = e."""
    main, comm = [], []
    for r in range(world):
        main.append(("write", rank, "param", r, ("p", 0, r)))      # identical initial parameters everywhere
    for e in range(1, steps + 1):
        if e > 1:
            for r in range(world):
                main.append(("wait", GATHERED, r, e - 1))
        for r in range(world):
            main.append(("read", rank, "param", r, ("p", e - 1, r)))
        for shard in range(world):
            main.append(("write", rank, "grad", shard, ("g", e, rank)))
        main.append(("set", "grads_final", e))
        comm.append(("need", "grads_final", e))
        for dst in range(world):
            comm.append(("signal", dst, READY, e))
        for r in range(world):
            comm.append(("wait", READY, r, e))
        for r in range(world):
            comm.append(("read", r, "grad", rank, ("g", e, r)))
        comm.append(("write", rank, "grad", rank, ("sum", e, rank)))
        for dst in range(world):
            comm.append(("signal", dst, DONE, e))
        comm.append(("set", "reduced", e))
        main.append(("need", "reduced", e))
        main.append(("read", rank, "grad", rank, ("sum", e, rank)))
        main.append(("write", rank, "param", rank, ("p", e, rank)))           # Adam writes the own shard
        main.append(("set", "adam", e))
        comm.append(("need", "adam", e))
        for d in range(1, world):
            comm.append(("write", (rank + d) % world, "param", rank, ("p", e, rank)))
        for dst in range(world):
            comm.append(("signal", dst, GATHERED, e))
        if wait_done_before_zero:
            for r in range(world):
                main.append(("wait", DONE, r, e))
        for shard in range(world):
            main.append(("write", rank, "grad", shard, ("zero", e, rank)))
    return {"main": main, "comm": comm}


def check(program, world, seeds=range(200), **kw):
    """Run ``program(world, rank, **kw)`` for all ranks under ``seeds`` random interleavings."""
    for seed in seeds:
        sim = Simulator(world)
        for rank in range(world):
            for name, ops in program(world, rank, **kw).items():
                sim.add(rank, name, ops)
        sim.run(seed)
