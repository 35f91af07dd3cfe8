"""Background batch assembly into pinned host memory.

One daemon thread runs ahead of the training loop by ``depth`` steps: it gathers the step's rows from the
memory-mapped streams into a ring of page-locked buffers (so the later host-to-device copy is a true
asynchronous DMA) and computes the host-side inner masks.  Delivery is checked to be in order
(reference ``src/ttt/data.py:880-909``).  A failure inside the thread is re-raised in the consumer.
"""
from __future__ import annotations

import queue
import threading
from typing import Optional, Tuple

import numpy as np
import torch


class Prefetcher:
    def __init__(self, sampler, start_step: int, depth: int = 4, mask_maker=None, pin: Optional[bool] = None):
        self.sampler, self.mask_maker = sampler, mask_maker
        self.depth = max(1, depth)
        pin = torch.cuda.is_available() if pin is None else pin
        self._ring = [torch.empty((sampler.local, sampler.T), dtype=torch.int32, pin_memory=pin) for _ in range(self.depth + 2)]
        self._q: "queue.Queue" = queue.Queue(maxsize=self.depth)
        self._next, self._stop = start_step, threading.Event()
        self._thread = threading.Thread(target=self._run, name="dttt-prefetch", daemon=True)
        self._thread.start()

    def _run(self) -> None:
        step, slot = self._next, 0
        try:
            while not self._stop.is_set():
                buf = self._ring[slot % len(self._ring)]
                ids = self.sampler.batch(step, out=buf.numpy())
                host = self.mask_maker(ids) if self.mask_maker is not None else None
                while not self._stop.is_set():
                    try:
                        self._q.put((step, buf, host), timeout=0.2)
                        break
                    except queue.Full:
                        continue
                step, slot = step + 1, slot + 1
        except BaseException as e:                                  # surfaced by get()
            self._q.put((-1, e, None))

    def get(self, step: int) -> Tuple[np.ndarray, Optional[np.ndarray]]:
        """``(ids [local, T] int32 numpy view of a pinned buffer, host mask or None)`` for ``step``."""
        s, buf, host = self._q.get()
        if s == -1:
            raise RuntimeError("prefetch thread failed") from buf
        if s != step:
            raise RuntimeError(f"prefetch out of order: got {s}, wanted {step}")
        return buf.numpy(), host

    def get_tensor(self, step: int):
        s, buf, host = self._q.get()
        if s == -1:
            raise RuntimeError("prefetch thread failed") from buf
        if s != step:
            raise RuntimeError(f"prefetch out of order: got {s}, wanted {step}")
        return buf, host

    def close(self) -> None:
        self._stop.set()
