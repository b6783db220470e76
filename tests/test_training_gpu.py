"""Whole-model training runs on one GPU (child processes, so each gets a fresh process group and CUDA context)."""
import os
import subprocess
import sys

import pytest

from common import ROOT, free_port


def _run(worker, marker, timeout=600):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), WORLD_SIZE="1", RANK="0",
               LOCAL_RANK="0")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "tests", "workers", worker)], env=env, capture_output=True,
                       text=True, timeout=timeout)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and marker in out, out[-4000:]


@pytest.mark.gpu
def test_fp16_training_with_overflow_recovery():
    """fp16 parameters on the native kernels (GEMM, flash attention, norms), dynamic loss scale: the oversized initial
    scale overflows, those steps are skipped without touching the parameters, the scale drops and the loss falls."""
    _run("fp16_smoke_worker.py", "FP16_SMOKE_OK")


@pytest.mark.gpu
def test_moe_grouped_kernels_match_the_per_expert_loop_and_train():
    """Fused router, dispatch, grouped tcgen05 GEMMs (forward, dgrad, wgrad) and combine against the per-expert loop
    (dropless and with a capacity limit), then a small MoE model trains through them."""
    _run("moe_grouped_worker.py", "MOE_GROUPED_OK")


@pytest.mark.gpu
def test_cuda_graph_decoding_matches_eager_decoding_and_is_faster():
    """Fixed-capacity key/value caches + one captured decoding step replayed per token (``cuda_graph_decode``)."""
    _run("graph_decode_worker.py", "GRAPH_DECODE_OK")
