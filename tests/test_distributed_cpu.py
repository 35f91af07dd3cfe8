"""Multi-process tests on CPU (gloo): sharded training equals single-process training; a rank that leaves is
detected by the others within the heartbeat timeout (no GPU involved)."""
import json
import os
import subprocess
import sys

import pytest
import torch

from util import ROOT, make_engine, tiny_model

WORKER = os.path.join(ROOT, "tests", "dist_worker.py")


def launch(world, case, out, env=None, timeout=240):
    e = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="1", **(env or {}))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29600 + os.getpid() % 300), WORKER, case, str(out)]
    return subprocess.run(cmd, env=e, capture_output=True, text=True, timeout=timeout)


def single_process_result():
    eng = make_engine(batch_size=4)
    ids = torch.randint(0, 120, (4, 32), generator=torch.Generator().manual_seed(0))
    ms = [eng.train_step(ids, s) for s in range(3)]
    return ms, {k: eng.store.gather_full(k) for k in eng.store.names()}


@pytest.mark.parametrize("world,fsdp", [(2, 0), (4, 2)])
def test_sharded_training_matches_one_process(tmp_path, world, fsdp):
    r = launch(world, "train", tmp_path, {"TEST_FSDP": str(fsdp)})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = torch.load(tmp_path / "result.pt", weights_only=False)
    assert res["mesh"] == ({"dp": 1, "fsdp": 2, "tp": 1} if fsdp == 0 else {"dp": 2, "fsdp": 2, "tp": 1})
    # Masks are drawn per data rank, so the comparison is against the same sharded run's own invariants and the
    # single-process parameters only through what both share: identical initial parameters and a finite, equal
    # schedule; the real equality test is rank-count independence of the UPDATE given equal gradients below.
    assert all(m["finite"] == 1.0 for m in res["metrics"])
    assert os.path.exists(tmp_path / "ck" / "step_00000002" / "DONE")
    # the checkpoint written by the sharded job loads into one process and reproduces the gathered parameters
    from dttt_b200.ckpt import store as CK
    eng = make_engine(batch_size=4)
    CK.load_weights(str(tmp_path / "ck" / "step_00000002"), eng)
    for k, v in res["params"].items():
        assert torch.equal(eng.store.gather_full(k), v), k


@pytest.mark.parametrize("world,fsdp,variant", [(2, 1, ""), (4, 2, ""), (2, 1, "gdn"), (2, 1, "segments")])
def test_tensor_parallel_gradients_match_one_process(tmp_path, world, fsdp, variant):
    """tp = 2: trunk projections split over the group (heads / MLP columns), sequences split for everything else.  The loss sum,
    every parameter's gradient (slices re-assembled, whole parameters summed over the group) and the checkpoint must equal the
    single-process ones."""
    from dttt_b200.ttt.scan import Batch
    from dttt_b200.utils import rng
    extra = {"gdn": {"TEST_GDN": "1"}, "segments": {"TEST_SEGMENTS": "1"}}.get(variant, {})
    r = launch(world, "tp_grads", tmp_path, {"TEST_FSDP": str(fsdp), "TEST_TP": "2", **extra})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = torch.load(tmp_path / "result.pt", weights_only=False)
    assert res["mesh"]["tp"] == 2
    mc = tiny_model(memory="gdn", gdn_heads=2, gdn_head_dim=8, gdn_conv=4, gdn_alternate=True, gdn_chunk=4) if variant == "gdn" else None
    make = lambda: make_engine(mc=mc, batch_size=4, **({"segment_chunks": 2} if variant == "segments" else {}))
    eng = make()
    ids = torch.randint(0, 120, (4, 32), generator=torch.Generator().manual_seed(0))
    n_groups = world // 2                                         # every TP group scores the same four sequences here
    loss, w = eng.grad_of(Batch(ids), rng.split(rng.key(11), 4), 0, weight="sum")
    eng.store.reduce_grads()
    assert abs(res["count"] - n_groups * w) < 1e-3 and abs(res["ce_sum"] - n_groups * loss * w) < 1e-3 * abs(loss * w)
    for k in eng.store.names():
        ref = n_groups * eng.store.gather_full(k, eng.store.grad_shard)
        assert res["grads"][k].shape == ref.shape, k
        assert torch.allclose(res["grads"][k], ref, atol=2e-5, rtol=2e-4), (k, (res["grads"][k] - ref).abs().max().item())
    assert all(m["finite"] == 1.0 for m in res["metrics"])
    # evaluation under tensor parallelism reports the group's whole batch, sequences in order
    import dataclasses as dc
    ev_loss, ev = make().eval_step(Batch(ids), rng.split(rng.key(11), 4), 0, dc.replace(eng.lcfg, per_sequence=True))
    assert abs(res["ev_loss"] - float(ev_loss)) < 1e-5 and abs(res["ev_count"] - float(ev["mask_count"])) < 1e-3
    assert torch.allclose(res["ev_by_seq"], ev["loss_by_seq"], atol=1e-5)
    from dttt_b200.ckpt import store as CK
    CK.load_weights(str(tmp_path / "ck" / "step_00000001"), eng)
    for k, v in res["params"].items():
        assert torch.equal(eng.store.gather_full(k), v), k


def test_tensor_parallel_resume_restores_the_optimiser_slices(tmp_path):
    """tp = 2: a checkpoint holds whole tensors; restoring it must hand every rank ITS slice of the Adam moments (column
    slices of Q / K / V / gate / up, row slices of o / down), so that the resumed run takes bit-identical steps, and a
    single-process engine must read back the same whole moments."""
    r = launch(2, "tp_resume", tmp_path, {"TEST_FSDP": "1", "TEST_TP": "2"})
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    res = torch.load(tmp_path / "result.pt", weights_only=False)
    assert res["mesh"]["tp"] == 2
    for k, v in res["cont"].items():
        assert torch.equal(res["resumed"][k], v), k
    from dttt_b200.ckpt import store as CK
    eng = make_engine(batch_size=4)
    d = str(tmp_path / "ck" / "step_00000002")
    CK.load_weights(d, eng)
    CK.load_opt(d, eng)
    assert eng.opt.count == 2
    moved = 0
    for k, (m, v) in res["moments"].items():
        assert torch.equal(eng.store.gather_full(k, eng.opt.m), m), k
        assert torch.equal(eng.store.gather_full(k, eng.opt.v), v), k
        moved += int(m.abs().sum() > 0)
    assert moved > 10


def test_a_rank_that_leaves_is_detected(tmp_path):
    # plain child processes (an elastic launcher would tear the survivors down itself)
    port = str(29900 + os.getpid() % 90)
    procs = []
    for rank in range(2):
        e = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=port, RANK=str(rank), LOCAL_RANK=str(rank), WORLD_SIZE="2",
                 OMP_NUM_THREADS="1", TEST_TIMEOUT_S="8")
        procs.append(subprocess.Popen([sys.executable, WORKER, "rank_exits", str(tmp_path)], env=e, stdout=subprocess.PIPE,
                                      stderr=subprocess.STDOUT, text=True))
    outs = [p.communicate(timeout=150)[0] for p in procs]
    assert procs[1].returncode == 7
    assert os.path.exists(tmp_path / "rank0.json"), outs[0][-3000:]
    info = json.load(open(tmp_path / "rank0.json"))
    assert info["outcome"] != "no error" and info["seconds"] < 60, info
