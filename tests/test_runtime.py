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
