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
