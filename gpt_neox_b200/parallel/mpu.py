"""Process-group bookkeeping for 3-D (+ expert) parallelism.

Rank layout follows the reference topology ``PipeModelDataParallelTopology(pp, mp, dp)`` with axes
ordered pipe -> data -> model (``megatron/initialize.py:166-170``), i.e.::

    global_rank = pipe_idx * (dp * mp) + data_idx * mp + model_idx

so tensor-parallel peers are adjacent ranks (same NVSwitch domain, lowest latency), data-parallel
peers are ``mp`` apart and pipeline neighbours ``dp * mp`` apart.  Groups built
(``megatron/mpu/initialize.py:53-159``): model (TP), data (DP), pipe (PP), io (first and last stage of
model-rank 0) and, for MoE, expert-parallel (EP) and expert-data-parallel groups carved out of DP.

When ``torch.distributed`` is not initialised (single process) every getter returns the trivial
answer (world size 1, rank 0, group ``None``) and collectives become no-ops, so a 1-GPU run needs no
rendezvous.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class Topology:
    """Cartesian rank grid with named axes, first axis slowest."""
    pp: int = 1
    dp: int = 1
    mp: int = 1

    @property
    def world_size(self):
        return self.pp * self.dp * self.mp

    def rank(self, pipe: int, data: int, model: int) -> int:
        return (pipe * self.dp + data) * self.mp + model

    def coords(self, rank: int):
        model = rank % self.mp
        data = (rank // self.mp) % self.dp
        pipe = rank // (self.mp * self.dp)
        return pipe, data, model

    def axis_lists(self, axis: str):
        """All groups of ranks that differ only along ``axis``."""
        out = []
        if axis == "model":
            for p in range(self.pp):
                for d in range(self.dp):
                    out.append([self.rank(p, d, m) for m in range(self.mp)])
        elif axis == "data":
            for p in range(self.pp):
                for m in range(self.mp):
                    out.append([self.rank(p, d, m) for d in range(self.dp)])
        elif axis == "pipe":
            for d in range(self.dp):
                for m in range(self.mp):
                    out.append([self.rank(p, d, m) for p in range(self.pp)])
        else:
            raise ValueError(axis)
        return out


@dataclass
class _State:
    initialized: bool = False
    topology: Topology = field(default_factory=Topology)
    rank: int = 0
    model_group: object = None
    data_group: object = None
    pipe_group: object = None
    io_group: object = None
    expert_group: object = None
    expert_data_group: object = None
    model_ranks: list = field(default_factory=lambda: [0])
    data_ranks: list = field(default_factory=lambda: [0])
    pipe_ranks: list = field(default_factory=lambda: [0])
    expert_ranks: list = field(default_factory=lambda: [0])
    expert_data_ranks: list = field(default_factory=lambda: [0])
    ep: int = 1
    fp32_allreduce: bool = False
    # overrides used by conversion / inspection tools
    mp_world_override: int | None = None
    mp_rank_override: int | None = None
    pipe_world_override: int | None = None
    pipe_rank_override: int | None = None


_S = _State()


def _dist_on() -> bool:
    return dist.is_available() and dist.is_initialized()


def initialize_model_parallel(model_parallel_size: int, pipe_parallel_size: int = 1, expert_parallel_size: int = 1,
                              topology: Topology | None = None, fp32_allreduce: bool = False):
    """Create every process group.  Must be called by all ranks with identical arguments."""
    global _S
    world = dist.get_world_size() if _dist_on() else 1
    rank = dist.get_rank() if _dist_on() else 0
    mp = min(max(model_parallel_size, 1), world)
    pp = max(pipe_parallel_size, 1)
    if topology is None:
        assert world % (mp * pp) == 0, f"world size {world} not divisible by mp*pp = {mp}*{pp}"
        topology = Topology(pp=pp, dp=world // (mp * pp), mp=mp)
    assert topology.world_size == world, f"topology {topology} does not cover world size {world}"
    s = _State(initialized=True, topology=topology, rank=rank, fp32_allreduce=fp32_allreduce)

    def make(lists, store_group, store_ranks):
        for ranks in lists:
            grp = dist.new_group(ranks) if _dist_on() else None
            if rank in ranks:
                setattr(s, store_group, grp)
                setattr(s, store_ranks, ranks)

    make(topology.axis_lists("data"), "data_group", "data_ranks")
    make(topology.axis_lists("pipe"), "pipe_group", "pipe_ranks")
    make(topology.axis_lists("model"), "model_group", "model_ranks")
    # io group: model-rank-0 processes of the first and last pipeline stage (they touch the data)
    io_ranks = sorted({topology.rank(p, d, 0) for p in {0, topology.pp - 1} for d in range(topology.dp)})
    grp = dist.new_group(io_ranks) if _dist_on() else None
    if rank in io_ranks:
        s.io_group = grp
    # expert parallel: consecutive blocks of `ep` ranks inside each data-parallel group
    ep = max(1, min(expert_parallel_size, topology.dp))
    assert topology.dp % ep == 0, f"data-parallel size {topology.dp} not divisible by expert-parallel size {ep}"
    s.ep = ep
    for dp_ranks in topology.axis_lists("data"):
        for i in range(0, len(dp_ranks), ep):
            ranks = dp_ranks[i:i + ep]
            grp = dist.new_group(ranks) if (_dist_on() and ep > 1) else None
            if rank in ranks:
                s.expert_group, s.expert_ranks = grp, ranks
        for j in range(ep):
            ranks = dp_ranks[j::ep]
            grp = dist.new_group(ranks) if (_dist_on() and ep > 1) else None
            if rank in ranks:
                s.expert_data_group, s.expert_data_ranks = grp, ranks
    if ep == 1:
        s.expert_data_group, s.expert_data_ranks = s.data_group, s.data_ranks
    _S = s
    return s


def model_parallel_is_initialized() -> bool:
    return _S.initialized


def destroy_model_parallel():
    global _S
    _S = _State()


def get_topology() -> Topology:
    return _S.topology


def get_fp32_allreduce() -> bool:
    return _S.fp32_allreduce


# ---------------------------------------------------------------- model (tensor) parallel
def get_model_parallel_group():
    return _S.model_group


def get_model_parallel_world_size() -> int:
    if _S.mp_world_override is not None:
        return _S.mp_world_override
    return len(_S.model_ranks)


def get_model_parallel_rank() -> int:
    if _S.mp_rank_override is not None:
        return _S.mp_rank_override
    return _S.model_ranks.index(_S.rank) if _S.rank in _S.model_ranks else 0


def set_model_parallel_world_size(n):
    _S.mp_world_override = n


def set_model_parallel_rank(r):
    _S.mp_rank_override = r


def get_model_parallel_src_rank() -> int:
    """Global rank of model-parallel rank 0 in this rank's TP group."""
    return _S.model_ranks[0]


def get_model_parallel_ranks():
    return list(_S.model_ranks)


# the Megatron-LM spellings of the same four (``megatron/mpu/initialize.py:274-298``)
def get_tensor_model_parallel_group():
    return get_model_parallel_group()


def get_tensor_model_parallel_src_rank() -> int:
    return get_model_parallel_src_rank()


def get_tensor_model_parallel_world_size() -> int:
    return get_model_parallel_world_size()


def get_tensor_model_parallel_rank() -> int:
    return get_model_parallel_rank()


def is_unitialized() -> bool:
    """For code that may run with or without the groups set up (the reference's spelling)."""
    return not _S.initialized


# ---------------------------------------------------------------- data parallel
def get_data_parallel_group():
    return _S.data_group


def get_data_parallel_world_size() -> int:
    return len(_S.data_ranks)


def get_data_parallel_rank() -> int:
    return _S.data_ranks.index(_S.rank) if _S.rank in _S.data_ranks else 0


def get_data_parallel_src_rank() -> int:
    return _S.data_ranks[0]


def get_data_parallel_ranks():
    return list(_S.data_ranks)


# ---------------------------------------------------------------- pipeline parallel
def get_pipe_parallel_group():
    return _S.pipe_group


def get_pipe_parallel_world_size() -> int:
    if _S.pipe_world_override is not None:
        return _S.pipe_world_override
    return len(_S.pipe_ranks)


def get_pipe_parallel_rank() -> int:
    if _S.pipe_rank_override is not None:
        return _S.pipe_rank_override
    return _S.pipe_ranks.index(_S.rank) if _S.rank in _S.pipe_ranks else 0


def set_pipe_parallel_world_size(n):
    _S.pipe_world_override = n


def set_pipe_parallel_rank(r):
    _S.pipe_rank_override = r


def get_pipe_parallel_ranks():
    return list(_S.pipe_ranks)


def is_pipeline_first_stage() -> bool:
    return get_pipe_parallel_rank() == 0


def is_pipeline_last_stage() -> bool:
    return get_pipe_parallel_rank() == get_pipe_parallel_world_size() - 1


def get_io_parallel_group():
    return _S.io_group


# ---------------------------------------------------------------- expert parallel
def get_expert_parallel_group():
    return _S.expert_group


def get_expert_parallel_world_size() -> int:
    return len(_S.expert_ranks)


def get_expert_parallel_rank() -> int:
    return _S.expert_ranks.index(_S.rank) if _S.rank in _S.expert_ranks else 0


def get_expert_parallel_ranks():
    return list(_S.expert_ranks)


def get_expert_data_parallel_group():
    return _S.expert_data_group


def get_expert_data_parallel_world_size() -> int:
    return len(_S.expert_data_ranks)


def get_expert_data_parallel_rank() -> int:
    return _S.expert_data_ranks.index(_S.rank) if _S.rank in _S.expert_data_ranks else 0


# ---------------------------------------------------------------- small helpers
def divide(numerator: int, denominator: int) -> int:
    assert numerator % denominator == 0, f"{numerator} is not divisible by {denominator}"
    return numerator // denominator


def split_tensor_along_last_dim(tensor, num_partitions, contiguous_split_chunks=False):
    size = divide(tensor.size(-1), num_partitions)
    parts = torch.split(tensor, size, dim=-1)
    return tuple(p.contiguous() for p in parts) if contiguous_split_chunks else parts


class VocabUtility:
    """Contiguous vocabulary range [first, last) owned by a tensor-parallel rank."""

    @staticmethod
    def vocab_range_from_per_partition_vocab_size(per_partition, rank, world_size):
        return rank * per_partition, (rank + 1) * per_partition

    @staticmethod
    def vocab_range_from_global_vocab_size(global_vocab_size, rank, world_size):
        return VocabUtility.vocab_range_from_per_partition_vocab_size(divide(global_vocab_size, world_size), rank,
                                                                      world_size)
