"""All-gather -> GEMM and GEMM -> reduce-scatter fused kernels on 2+ GPUs (one process per GPU, peer memory over NVLink)."""
import os
import subprocess
import sys

import pytest
import torch

from util import ROOT

pytestmark = pytest.mark.gpu


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_column_and_row_parallel_linear_match_unsharded():
    n = 2 if torch.cuda.device_count() < 4 else 4
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29720", os.path.join(ROOT, "tests", "tp_worker.py")]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=dict(os.environ, NCCL_NVLS_ENABLE="0"))
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "TP_WORST_REL_ERR" in r.stdout


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_tensor_parallel_model_matches_one_gpu(tmp_path):
    """The whole training loss (second order through the write) with tp = 2 on the fused kernels against one GPU."""
    worker = os.path.join(ROOT, "tests", "tp_model_worker.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, worker, str(tmp_path), "1"], capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29730", worker, str(tmp_path), "2"]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    a = torch.load(tmp_path / "tp1.pt", weights_only=False)
    b = torch.load(tmp_path / "tp2.pt", weights_only=False)
    assert b["finite"] == 1.0
    assert abs(a["count"] - b["count"]) < 1e-3
    assert abs(a["ce_sum"] - b["ce_sum"]) < 1e-2 * abs(a["ce_sum"])
    cos = torch.nn.functional.cosine_similarity
    for k in a["grads"]:
        ga, gb = a["grads"][k].flatten().double(), b["grads"][k].flatten().double()
        assert ga.shape == gb.shape, k
        if ga.norm() > 1e-6:
            assert cos(ga, gb, dim=0).item() > 0.98, (k, cos(ga, gb, dim=0).item())
            assert abs(ga.norm() - gb.norm()) < 0.1 * ga.norm(), k
