"""The training entry point as a user runs it (subprocess CLI): bitwise resume, refused data change, init_from,
continue_from, triggers (the reference's tests/test_train_smoke.py and tests/test_trigger.py are the model)."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from util import ROOT
from dttt_b200.ckpt import npystream as NS
from dttt_b200.data.synth import write_stream, zipf_tokens


@pytest.fixture(scope="module")
def work(tmp_path_factory):
    d = tmp_path_factory.mktemp("cli")
    for i, n in enumerate(("a", "b")):
        write_stream(str(d / "data" / n), zipf_tokens(120_000, 1024, seed=i, eos=1022, mean_doc=150), 1022, n, 1024)
    run = {"model_config": os.path.join(ROOT, "configs/tiny_baseline"), "data_root": str(d / "data"), "sources": "a=a:0.6,b=b:0.4",
           "seq_len": 256, "batch_size": 2, "grad_accum": 2, "steps": 6, "seed": 0, "lr": 0.001, "warmup_steps": 2,
           "inner_lr_warmup_steps": 2, "inner_task": "causal", "outer_shift": True, "cart_window": 32, "holdout": 20000,
           "eval_batches": 1, "eval_interval": 100, "eval_step0": False, "ckpt_interval": 3, "keep_checkpoints": 0, "log_interval": 1,
           "fused_ce_block": 0, "compute_dtype": "float32"}
    (d / "run.json").write_text(json.dumps(run))
    return d


def train(work, *flags, env=None):
    cmd = [sys.executable, "-m", "dttt_b200.train", "--config", str(work / "run.json"), *map(str, flags)]
    return subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600, env=dict(os.environ, OMP_NUM_THREADS="2", **(env or {})))


def leaves(step_dir):
    return list(NS.read_records(os.path.join(step_dir, "model.eqx"))) + list(NS.read_records(os.path.join(step_dir, "opt.eqx")))


def test_six_steps_equal_three_plus_resume_three_bitwise(work):
    r = train(work, "--ckpt_dir", work / "full")
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "[      5] loss" in r.stdout and "checkpoint ->" in r.stdout
    r1 = train(work, "--ckpt_dir", work / "split", "--steps", 3)
    assert r1.returncode == 0, r1.stderr[-2000:]
    r2 = train(work, "--ckpt_dir", work / "split", "--resume", "auto")
    assert r2.returncode == 0 and "resumed" in r2.stdout and "resume data check" in r2.stdout, r2.stdout[-2000:] + r2.stderr[-2000:]
    a, b = leaves(work / "full" / "step_00000005"), leaves(work / "split" / "step_00000005")
    assert len(a) == len(b) and all(np.array_equal(x, y) for x, y in zip(a, b))
    # run again: nothing left to do, stops at once
    r3 = train(work, "--ckpt_dir", work / "split", "--resume", "auto")
    assert r3.returncode == 0 and "[      5] loss" not in r3.stdout


def test_resume_refuses_a_changed_data_configuration(work):
    r = train(work, "--ckpt_dir", work / "full", "--resume", "auto", "--steps", 8, "--seed", 1)
    assert r.returncode != 0 and "data configuration changed" in (r.stdout + r.stderr)


def test_init_from_and_continue_from(work):
    src = work / "full" / "step_00000005"
    r = train(work, "--ckpt_dir", work / "init", "--init_from", src, "--steps", 2, "--ckpt_interval", 0)
    assert r.returncode == 0 and "initialised weights from" in r.stdout and "[      0] loss" in r.stdout
    r = train(work, "--ckpt_dir", work / "branch", "--continue_from", src, "--steps", 8)
    assert r.returncode == 0 and "continuing" in r.stdout and "[      6] loss" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
    assert json.load(open(work / "branch" / "step_00000007" / "state.json"))["data_offset"] == 0      # same stream, read on
    r = train(work, "--ckpt_dir", work / "full", "--continue_from", src)
    assert r.returncode != 0 and "ckpt_dir of its own" in (r.stdout + r.stderr)


def test_trigger_stop_writes_a_checkpoint_and_exits(work):
    trig = work / "trig"
    trig.mkdir()
    p = subprocess.Popen([sys.executable, "-m", "dttt_b200.train", "--config", str(work / "run.json"), "--ckpt_dir", str(work / "trigrun"),
                          "--steps", "400", "--ckpt_interval", "0"], cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                         env=dict(os.environ, OMP_NUM_THREADS="2", DTTT_TRIGGER_DIR=str(trig)))
    seen = ""
    for line in p.stdout:
        seen += line
        if "[      2] loss" in line:
            (trig / "TRIGGER_STOP").write_text("")
        if "triggered stop" in line:
            break
    p.wait(timeout=120)
    assert p.returncode == 0 and "triggered checkpoint" in seen and "triggered stop" in seen, seen[-2000:]
    assert not (trig / "TRIGGER_STOP").exists()
    assert any(d.startswith("step_") for d in os.listdir(work / "trigrun"))


def test_probe_memory_and_flags_parse(work):
    r = train(work, "--probe_memory", "true", "--ckpt_dir", work / "pm")
    assert r.returncode == 0
    r = train(work, "--steps", 1, "--ckpt_interval", 0, "--inner_mask_range", 0.3, 0.6, "--inner_task", "mask", "--outer_shift", "false",
              "--ckpt_dir", work / "flags")
    assert r.returncode == 0 and "inner_mask_range=(0.3, 0.6)" in r.stdout, r.stdout[-1500:] + r.stderr[-1500:]
