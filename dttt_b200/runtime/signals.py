"""Operator controls of a running job: ask for a checkpoint, or for a checkpoint and a clean exit.

Two channels, merged: marker files in a watched directory (``TRIGGER_SAVE`` / ``TRIGGER_STOP``; the directory is
``$DTTT_TRIGGER_DIR``, else ``$TTT_TRIGGER_DIR``, else ``./log``) and the signals SIGUSR1 (save) / SIGUSR2 (stop).  The training
loop asks once per step; with several ranks the requests are max-reduced, so one host's file or signal is enough.  The reference
offers the same controls (src/ttt/train.py:49-91).
"""
from __future__ import annotations

import enum
import os
import signal
from typing import Optional

import torch


class Request(enum.IntEnum):
    NONE = 0
    SAVE = 1
    STOP = 2


def default_directory() -> str:
    return os.environ.get("DTTT_TRIGGER_DIR") or os.environ.get("TTT_TRIGGER_DIR") or os.path.join(os.getcwd(), "log")


class OperatorSignals:
    FILES = {"TRIGGER_SAVE": Request.SAVE, "TRIGGER_STOP": Request.STOP}

    def __init__(self, directory: Optional[str] = None, install_handlers: bool = True):
        self.directory = directory or default_directory()
        self._by_signal = Request.NONE
        if install_handlers:
            for signum, req in ((signal.SIGUSR1, Request.SAVE), (signal.SIGUSR2, Request.STOP)):
                try:
                    signal.signal(signum, self._handler(req))
                except (ValueError, OSError):            # not the main thread, or a platform without the signal
                    pass

    def _handler(self, req: Request):
        def on_signal(_signum, _frame):
            self._by_signal = max(self._by_signal, req)
        return on_signal

    def pending(self) -> Request:
        """The strongest request seen on this host since the last ``clear``."""
        req = self._by_signal
        for name, r in self.FILES.items():
            if os.path.exists(os.path.join(self.directory, name)):
                req = max(req, r)
        return Request(req)

    def agreed(self, device: torch.device, world: int) -> Request:
        """``pending`` max-reduced over the job (every rank must call it in the same step)."""
        req = int(self.pending())
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([req], device=device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            req = int(t.item())
        return Request(req)

    def clear(self) -> None:
        self._by_signal = Request.NONE
        for name in self.FILES:
            try:
                os.remove(os.path.join(self.directory, name))
            except OSError:
                pass
