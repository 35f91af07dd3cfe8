"""The pieces a run is assembled from (``dttt_b200.runtime``): operator signals, command line -> configuration, write plans."""
import json
import os
import signal

import pytest
import torch

from dttt_b200.runtime import cliargs, evalsuite
from dttt_b200.runtime.signals import OperatorSignals, Request


def test_operator_requests_merge_files_and_signals(tmp_path):
    sig = OperatorSignals(str(tmp_path))
    assert sig.pending() == Request.NONE
    (tmp_path / "TRIGGER_SAVE").write_text("")
    assert sig.pending() == Request.SAVE
    os.kill(os.getpid(), signal.SIGUSR2)
    assert sig.pending() == Request.STOP and sig.agreed(torch.device("cpu"), 1) == Request.STOP
    sig.clear()
    assert sig.pending() == Request.NONE and not (tmp_path / "TRIGGER_SAVE").exists()
    os.kill(os.getpid(), signal.SIGUSR1)
    assert sig.pending() == Request.SAVE
    (tmp_path / "TRIGGER_STOP").write_text("")
    assert sig.pending() == Request.STOP
    sig.clear()


def test_flags_override_the_run_file_and_numbers_take_the_fields_type(tmp_path):
    run = tmp_path / "run.json"
    run.write_text(json.dumps({"# note": "comment keys are skipped", "lr": 1, "steps": 40.0, "seq_len": 512, "outer_shift": True,
                               "inner_mask_range": [0.25, 0.75]}))
    cfg = cliargs.train_config_from_argv(["--config", str(run), "--seq_len", "1024", "--second_order", "no"])
    assert cfg.lr == 1.0 and isinstance(cfg.lr, float) and cfg.steps == 40 and isinstance(cfg.steps, int)
    assert cfg.seq_len == 1024 and cfg.outer_shift is True and cfg.second_order is False
    assert cfg.inner_mask_range == (0.25, 0.75)
    with pytest.raises(SystemExit):
        cliargs.train_config_from_argv(["--no_such_flag", "1"])


def test_write_plan_spec():
    assert evalsuite.parse_write_plan("", 4) == ()
    assert evalsuite.parse_write_plan("1:3, 2:0", 4) == (1, 3, 0, 1)
    with pytest.raises(ValueError):
        evalsuite.parse_write_plan("4:2", 4)


def test_refused_option_combinations():
    """``ttt.validate``: the table of combinations the objective refuses, and a few that it accepts."""
    import dataclasses as dc
    from util import loss_config, make_engine, tiny_model
    from dttt_b200.ttt import validate as VAL
    eng = make_engine()
    lc, mc = loss_config(eng.tc), eng.mc
    has_all, has_none = (lambda name: True), (lambda name: False)
    VAL.check_options(lc, mc, has_none)                                                     # the default objective is fine
    VAL.check_options(dc.replace(lc, mtp=True, outer_shift=True, inner_task="causal"), mc, has_all)
    refused = [dc.replace(lc, outer_views=0), dc.replace(lc, outer_views=2, per_token=True),
               dc.replace(lc, distill=True, no_write=True), dc.replace(lc, write_off=True, inner_views=2),
               dc.replace(lc, aux_causal_weight=0.5, no_write=True), dc.replace(lc, write_plan=(1, 2, 1, 1), inner_task="mask"),
               dc.replace(lc, write_plan=(1, -1, 1, 1)), dc.replace(lc, self_prior=0.1, no_write=True),
               dc.replace(lc, mtp=True, outer_shift=False), dc.replace(lc, reread_chunks=2, segment_chunks=0),
               dc.replace(lc, reread_chunks=3, segment_chunks=2), dc.replace(lc, inner_feat="cos", no_write=True)]
    for bad in refused:
        with pytest.raises(ValueError):
            VAL.check_options(bad, mc, has_all)
    with pytest.raises(ValueError):                                                         # a head the model was not built with
        VAL.check_options(dc.replace(lc, mtp=True, outer_shift=True, inner_task="causal"), mc, has_none)
    with pytest.raises(ValueError):
        VAL.check_options(dc.replace(lc, no_write=True), mc, has_all, use_gdn=True, gdn_requested={"distill": True})
    assert VAL.check_geometry(64, mc, 0, 8) == 8 and VAL.check_geometry(64, mc, 4, 8) == 4
    for args in ((60, mc, 0, 7), (64, mc, 3, 8), (64, tiny_model(window_chunks=3), 2, 8)):
        with pytest.raises(ValueError):
            VAL.check_geometry(*args)


def test_keep_knobs_below_zero_are_filled_in_from_the_memory_model():
    from dttt_b200.engine import resolve_keep
    from dttt_b200.schema import ModelConfig, TrainConfig
    from util import ROOT
    mc = ModelConfig.load(os.path.join(ROOT, "configs/b200_1b_8k"))
    tc = TrainConfig(model_config="configs/b200_1b_8k", seq_len=8192, batch_size=2, keep_prefix_layers=-1, keep_suffix_chunks=-1)
    roomy = resolve_keep(tc, mc, 154e9, 2)                     # a B200 after the parameters: everything fits (measured: 129 GB peak)
    assert (roomy.keep_prefix_layers, roomy.keep_suffix_chunks) == (12, 8)
    tight = resolve_keep(tc, mc, 90e9, 2)
    assert tight.keep_suffix_chunks == 8 and 0 <= tight.keep_prefix_layers < 12
    none = resolve_keep(tc, mc, 40e9, 2)
    assert (none.keep_prefix_layers, none.keep_suffix_chunks) == (0, 0)
    four = resolve_keep(tc, mc, 154e9, 4)                      # four sequences per pass: only part of it fits
    assert four.keep_suffix_chunks + four.keep_prefix_layers < 20 and four.keep_suffix_chunks >= 1
    fixed = resolve_keep(tc.replace(keep_suffix_chunks=3), mc, 154e9, 2)
    assert fixed.keep_suffix_chunks == 3 and fixed.keep_prefix_layers == 12
    assert resolve_keep(tc.replace(keep_prefix_layers=0, keep_suffix_chunks=0), mc, 0.0, 2).keep_prefix_layers == 0
    # 32k, one sequence per pass, the method arm (normalised write + self-prior): a kept chunk step costs about twice the plain
    # one, and the plan must stay inside what was measured to fit (four steps per segment: 126 GiB; eight: out of memory)
    mc32 = ModelConfig.load(os.path.join(ROOT, "configs/b200_1b_32k"))
    long_ = TrainConfig(model_config="configs/b200_1b_32k", seq_len=32768, batch_size=1, segment_chunks=8, keep_prefix_layers=-1,
                        keep_suffix_chunks=-1, inner_task="causal", outer_shift=True)
    plain = resolve_keep(long_, mc32, 160e9, 1)
    method = resolve_keep(long_.replace(inner_norm_alpha=1.0, inner_norm_cap=128.0, self_prior=0.1), mc32, 160e9, 1)
    assert plain.keep_suffix_chunks == 8 and 3 <= method.keep_suffix_chunks <= 6
