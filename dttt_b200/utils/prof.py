"""Device-time accounting by label.

``with prof.range("label"):`` brackets a region with two CUDA events on the current stream when
profiling is on (``DTTT_PROFILE=1`` or ``prof.enable()``); ``prof.report()`` synchronises once and returns
the accumulated milliseconds and call counts per label.  Nested ranges are allowed (their times overlap).
Off by default: the context manager is then a no-op.  This is the in-process counterpart of the
reference's profiler trace hooks (``src/ttt/train.py:1096-1107``): it gives per-phase device time without
an external profiler attached.
"""
from __future__ import annotations

import contextlib
import os
from collections import defaultdict
from typing import Dict, List, Tuple

import torch

_ON = os.environ.get("DTTT_PROFILE", "0") == "1"
_events: List[Tuple[str, torch.cuda.Event, torch.cuda.Event]] = []


def enable(on: bool = True) -> None:
    global _ON
    _ON = on


def enabled() -> bool:
    return _ON


@contextlib.contextmanager
def range(label: str):
    if not _ON or not torch.cuda.is_available():
        yield
        return
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    try:
        yield
    finally:
        e1.record()
        _events.append((label, e0, e1))


def report(reset: bool = True) -> Dict[str, Tuple[float, int]]:
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    acc: Dict[str, List[float]] = defaultdict(lambda: [0.0, 0])
    for label, e0, e1 in _events:
        acc[label][0] += e0.elapsed_time(e1)
        acc[label][1] += 1
    if reset:
        _events.clear()
    return {k: (v[0], v[1]) for k, v in acc.items()}


def format_report(rep: Dict[str, Tuple[float, int]]) -> str:
    rows = sorted(rep.items(), key=lambda kv: -kv[1][0])
    return "\n".join(f"{k:40s} {ms:10.1f} ms  n={n}" for k, (ms, n) in rows)
