"""Fused GEMM + collective kernels over peer memory, on 2 GPUs (or more) of one node.

The checks live in ``tests/workers/fused_comm_worker.py`` (one process per GPU under torchrun): every fused op is
compared with the NCCL collective + fp32 matmul statement of the same math, over several iterations so both buffer
parities are reused, then a column->row parallel layer pair is run forward and backward both ways, and finally a wait
on an epoch nobody publishes must time out with a status code and leave the context usable.
"""
import json
import os
import subprocess
import sys

import pytest
import torch

from common import ROOT, free_port


@pytest.mark.gpu
@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_comm_kernels(world):
    n = torch.cuda.device_count()
    if n < world:
        pytest.skip(f"needs at least {world} GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "workers", "fused_comm_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "FUSED_COMM_OK" in out, out[-4000:]


@pytest.mark.gpu
def test_zero1_overlap_two_gpus():
    """Data-parallel ZeRO-1 on 2 GPUs: overlapped bucketed reduce-scatter / async all-gather == reduce-at-step."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "workers", "dp_overlap_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "DP_OVERLAP_OK" in out, out[-4000:]


@pytest.mark.gpu
def test_moe_peer_all_to_all_two_gpus():
    """Expert-parallel MoE on 2 GPUs: token exchange by peer-memory kernels == NCCL all-to-all (fwd and bwd)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs at least 2 GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
           os.path.join(ROOT, "tests", "workers", "moe_worker.py")]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "MOE_A2A_OK" in out, out[-4000:]


@pytest.mark.gpu
def test_tensor_parallel_training_parity(tmp_path):
    """The same model, data and host-drawn initial weights trained for ten steps at tensor-parallel degree 1, 2 and
    (with four GPUs) 4, through the fused compute+collective kernels, through the NCCL mappings and with sequence
    parallelism: every run must follow the degree-1 losses to bf16 accuracy."""
    n = torch.cuda.device_count()
    if n < 2:
        pytest.skip("needs at least 2 GPUs")
    results = {}
    for world in [w for w in (1, 2, 4) if w <= n]:
        out = str(tmp_path / f"tp{world}.json")
        env = dict(os.environ, NCCL_NVLS_ENABLE="0", TP_PARITY_OUT=out)
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
               "--master-addr", "127.0.0.1", "--master-port", str(free_port()),
               os.path.join(ROOT, "tests", "workers", "tp_parity_worker.py")]
        r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0 and "TP_PARITY_DONE" in r.stdout, (r.stdout + r.stderr)[-4000:]
        results[world] = json.load(open(out))
    base = results[1]["nccl"]
    assert base[-1] < base[0] - 0.05, base                  # it trains
    for world, runs in results.items():
        for name, losses in runs.items():
            worst = max(abs(a - b) for a, b in zip(losses, base))
            assert worst < 0.06, f"tp{world} {name}: {losses} vs tp1 {base}"
