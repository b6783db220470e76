"""Broadcast a dict of same-dtype tensors from tensor-parallel rank 0 to its TP group.

Reference ``megatron/mpu/data.py:35-120`` sends a size header and then one flattened payload.  Same
protocol here; with a TP world size of 1 the tensors are only moved to the compute device.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import mpu

_MAX_DIM = 4


def _device():
    return torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")


def broadcast_data(keys, data, datatype):
    dev = _device()
    tp = mpu.get_model_parallel_world_size()
    if tp == 1:
        return {k: data[k].to(device=dev, dtype=datatype, non_blocking=True) for k in keys}
    src, grp = mpu.get_model_parallel_src_rank(), mpu.get_model_parallel_group()
    header = torch.zeros(len(keys) * _MAX_DIM, dtype=torch.int64, device=dev)
    if mpu.get_model_parallel_rank() == 0:
        sizes = []
        for k in keys:
            assert data[k].dim() <= _MAX_DIM, "you should increase MAX_DATA_DIM"
            sizes.extend(list(data[k].shape) + [0] * (_MAX_DIM - data[k].dim()))
        header.copy_(torch.tensor(sizes, dtype=torch.int64))
    dist.broadcast(header, src, group=grp)
    hdr = header.tolist()
    shapes, total = {}, 0
    for i, k in enumerate(keys):
        shp = [d for d in hdr[i * _MAX_DIM:(i + 1) * _MAX_DIM] if d > 0]
        shapes[k] = shp
        n = 1
        for d in shp:
            n *= d
        total += n
    if mpu.get_model_parallel_rank() == 0:
        for k in keys:
            assert data[k].dtype == datatype, f"{k} has dtype {data[k].dtype}, expected {datatype}"
        flat = torch.cat([data[k].contiguous().view(-1) for k in keys]).to(dev)
    else:
        flat = torch.empty(total, dtype=datatype, device=dev)
    dist.broadcast(flat, src, group=grp)
    out, off = {}, 0
    for k in keys:
        n = 1
        for d in shapes[k]:
            n *= d
        out[k] = flat[off:off + n].view(shapes[k])
        off += n
    return out
