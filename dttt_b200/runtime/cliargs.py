"""Command line -> ``TrainConfig``.

Every field of the dataclass is a flag of the same name; ``--config FILE`` reads a run configuration first (``schema.load_run_config``:
JSON of the same fields, ``base`` inheritance, ``#`` comments) and flags given on the command line replace its values, as in the
reference (src/ttt/train.py:97-131).  Booleans take ``1/true/yes``; pair-valued fields take two numbers.
"""
from __future__ import annotations

import argparse
import dataclasses as dc
from typing import Any, Optional, Sequence

from ..schema import TrainConfig, load_run_config

PAIR_FIELDS = ("inner_mask_range", "distill_t_range")


def _as_bool(text: str) -> bool:
    return text.strip().lower() in ("1", "true", "yes")


def _match_type(default: Any, value: Any) -> Any:
    """JSON numbers arrive as int or float regardless of the field: 1 for a float field, 2.0 for an int field."""
    if isinstance(default, bool) or isinstance(value, bool):
        return value
    if isinstance(default, float) and isinstance(value, int):
        return float(value)
    if isinstance(default, int) and isinstance(value, float) and value.is_integer():
        return int(value)
    return value


def _config_file(argv: Optional[Sequence[str]]) -> str:
    first = argparse.ArgumentParser(add_help=False)
    first.add_argument("--config", default="")
    return first.parse_known_args(argv)[0].config


def build_parser(prog: str = "python -m dttt_b200.train") -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog=prog, formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("--config", default="", help="run configuration (JSON of these fields; 'base' inherits)")
    for field in dc.fields(TrainConfig):
        flag, default = f"--{field.name}", field.default
        if isinstance(default, bool):
            ap.add_argument(flag, type=_as_bool, default=default, dest=field.name)
        elif isinstance(default, tuple):
            ap.add_argument(flag, type=type(default[0]), nargs=len(default), default=default, dest=field.name,
                            metavar=("LO", "HI") if len(default) == 2 else None)
        else:
            ap.add_argument(flag, type=type(default), default=default, dest=field.name)
    return ap


def train_config_from_argv(argv: Optional[Sequence[str]] = None) -> TrainConfig:
    ap = build_parser()
    run_file = _config_file(argv)
    if run_file:
        declared = {f.name: f.default for f in dc.fields(TrainConfig)}
        ap.set_defaults(**{k: _match_type(declared[k], v) for k, v in load_run_config(run_file).items()})
    values = vars(ap.parse_args(argv))
    values.pop("config")
    for name in PAIR_FIELDS:
        values[name] = tuple(values[name])
    return TrainConfig(**values)
