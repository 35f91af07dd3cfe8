"""The benchmark's output contract, on the CPU: ``bench.py --config tiny`` (the small CPU configuration) prints one JSON
line with the agreed keys, and the reference arm answers with a number or with one ``unavailable`` line and exit code 0."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], cwd=ROOT, env=env, capture_output=True, text=True,
                       timeout=900)
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    return r, lines


def test_tiny_configuration_prints_the_agreed_line():
    r, lines = _run("--config", "tiny", "--steps", "1", "--warmup", "3")
    assert r.returncode == 0, r.stderr[-2000:]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "gpu_launches"):
        assert key in d, key
    assert d["steps"] == 1 and d["warmup"] == 3 and d["higher_is_better"] is True and d["value"] > 0
    assert abs(d["value"] - d["config"]["global_batch"] * d["config"]["seq_len"] / (d["ms_per_step"] / 1e3)) < 1e-6 * d["value"]
    assert d["device"] == "cpu" and d["gpu_launches"] == 0 and "synthetic" in d["data"]


def test_reference_arm_answers_in_one_line():
    r, lines = _run("--impl", "reference", "--steps", "1", "--warmup", "3")
    assert r.returncode == 0, r.stderr[-2000:]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and ("unavailable" in d or d.get("value", 0) > 0)
