"""FSDP weight all-gather fused into the consuming GEMM: the kernel against torch on 2+ GPUs, and a training run with
``shard_compute`` against the replicated layout."""
import os
import subprocess
import sys

import pytest
import torch

from util import ROOT

pytestmark = pytest.mark.gpu


def _run(n, port, worker, *args):
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", str(port), os.path.join(ROOT, "tests", worker), *args]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_gather_fused_gemm_matches_torch():
    out = _run(min(4, torch.cuda.device_count()), 29740, "wg_worker.py")
    assert "WG_WORST_REL_ERR" in out


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_shard_compute_training_matches_the_replicated_layout(tmp_path):
    """Three optimiser steps with the prefix matrices gathered per use (and every foreign part of the compute buffer
    poisoned) against the same run with replicated compute copies."""
    n = min(4, torch.cuda.device_count())
    _run(n, 29741, "fused_worker.py", str(tmp_path), "1")
    _run(n, 29742, "fused_worker.py", str(tmp_path), "shard")
    a = torch.load(tmp_path / "fused1.pt", weights_only=False)
    b = torch.load(tmp_path / "fusedshard.pt", weights_only=False)
    assert b["gather_launches"] > 0
    for s in range(3):
        la, lb = a["metrics"][s]["loss"], b["metrics"][s]["loss"]
        assert lb == lb and abs(la - lb) < 2e-3 * abs(la), (s, la, lb)
    g0a, g0b = a["metrics"][0]["grad_norm"], b["metrics"][0]["grad_norm"]
    assert abs(g0a - g0b) < 1e-3 * g0a, (g0a, g0b)
    for k in a["params"]:
        d = (a["params"][k] - b["params"][k]).abs()
        assert torch.isfinite(b["params"][k]).all(), k
        assert d.mean().item() < 1e-4 and d.max().item() < 3e-3, (k, d.mean().item(), d.max().item())
