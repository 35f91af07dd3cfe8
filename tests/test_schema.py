import json
import os

import pytest

from util import ROOT
from dttt_b200.schema import ModelConfig, TrainConfig, load_run_config


def test_unknown_key_is_an_error(tmp_path):
    p = tmp_path / "config.json"
    d = json.load(open(os.path.join(ROOT, "configs/tiny_smoke/config.json")))
    d["hiden_size"] = 3
    p.write_text(json.dumps(d))
    with pytest.raises(ValueError, match="unknown keys"):
        ModelConfig.load(str(p))


def test_retired_options_load_only_when_off(tmp_path):
    p = tmp_path / "run.json"
    p.write_text(json.dumps({"inner_assoc_scale": 1.0, "self_prior_delay": [0, 0], "seq_len": 64}))
    assert load_run_config(str(p)) == {"seq_len": 64}
    p.write_text(json.dumps({"inner_prior_k": 3}))
    with pytest.raises(ValueError, match="removed options in use"):
        load_run_config(str(p))


def test_base_chain_comments_and_cycles(tmp_path):
    (tmp_path / "a.json").write_text(json.dumps({"#": "note", "seq_len": 64, "lr": 0.5, "#lr": "why"}))
    (tmp_path / "b.json").write_text(json.dumps({"base": "a.json", "lr": 0.25}))
    (tmp_path / "c.json").write_text(json.dumps({"base": ["b.json", "a.json"], "steps": 7}))
    assert load_run_config(str(tmp_path / "b.json")) == {"seq_len": 64, "lr": 0.25}
    assert load_run_config(str(tmp_path / "c.json")) == {"seq_len": 64, "lr": 0.5, "steps": 7}
    (tmp_path / "x.json").write_text(json.dumps({"base": "y.json"}))
    (tmp_path / "y.json").write_text(json.dumps({"base": "x.json"}))
    with pytest.raises(ValueError, match="cycle"):
        load_run_config(str(tmp_path / "x.json"))


@pytest.mark.parametrize("name", sorted(os.listdir(os.path.join(ROOT, "runs"))))
def test_shipped_run_configs_load(name):
    d = load_run_config(os.path.join(ROOT, "runs", name))
    d = {k: tuple(v) if isinstance(v, list) else v for k, v in d.items()}
    if "continue_from" in d or name.startswith("stage_"):
        d.pop("continue_from", None)
    TrainConfig(**d)


def test_reference_run_configs_load_unchanged():
    tree = os.environ.get("DTTT_REFERENCE_TREE", "")          # a checkout of the reference, when one is at hand
    ref = os.path.join(tree, "runs")
    if not tree or not os.path.isdir(ref):
        pytest.skip("no reference checkout named by DTTT_REFERENCE_TREE")
    for f in os.listdir(ref):
        load_run_config(os.path.join(ref, f))
    ModelConfig.load(os.path.join(tree, "configs/1b_e2e"))
    ModelConfig.load(os.path.join(tree, "configs/tiny_smoke"))


def test_model_validation_and_derived():
    c = ModelConfig.load(os.path.join(ROOT, "configs/1b_e2e"))
    assert (c.prefix_len, c.fast_len, c.window_len, c.reach) == (18, 6, 3072, None)
    c2 = c.replace(suffix_len=12, suffix_plain_top=6)
    assert c2.fast_mask == (True,) * 6 + (False,) * 6 and c2.suffix_runs == ((True, 0, 6), (False, 6, 12))
    c3 = c.replace(suffix_len=8, fast_layers=[16, 18, 21])
    assert c3.fast_layer_indices == (16, 18, 21)
    with pytest.raises(ValueError):
        c.replace(fast_layers=[17, 18])
    with pytest.raises(ValueError):
        c.replace(memory="gdn", inner_lr_gate=True)
    with pytest.raises(ValueError):
        c.replace(read_block=100)
    rs = {"rope_type": "llama3", "factor": 16.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0, "original_max_position_embeddings": 8192}
    assert dict(c.replace(rope_scaling=rs).rope_scaling)["factor"] == 16.0


def test_train_validation_and_roundtrip(tmp_path):
    with pytest.raises(ValueError):
        TrainConfig(inner_subchunks=2, inner_task="mask")
    with pytest.raises(ValueError):
        TrainConfig(self_prior=0.1, no_write=True)
    with pytest.raises(ValueError):
        TrainConfig(decay_start=10, decay_end=5)
    with pytest.raises(ValueError):
        TrainConfig(resume="/x", init_from="/y")
    t = TrainConfig(inner_mask_range=(0.2, 0.9), tp_size=2)
    p = tmp_path / "t.json"
    t.save(str(p))
    assert TrainConfig.load(str(p)) == t
    d = json.load(open(p))
    assert "fused_comm" not in d and d["tp_size"] == 2        # additions are written only when changed
