"""ctypes loader of the in-tree CUDA library, plus the per-device status word.

The kernels report trouble (a bounded wait that gave up) through an ``int`` in device memory instead
of trapping; ``check_status()`` reads it (one small device-to-host copy) and raises.  Training code
calls it once per step, tests after each kernel.

On a machine with a GPU the library MUST load: a missing or unloadable ``.so`` raises at the first
kernel call instead of silently falling back to PyTorch ops.
"""
from __future__ import annotations

import ctypes
import os
import threading

import torch

from .. import build as _build

_lock = threading.Lock()
_lib = None
_status: dict[int, torch.Tensor] = {}

ERR_NAMES = {0: "ok", 1: "wait for a TMA stage (full barrier) timed out", 2: "wait for a free stage (empty barrier) timed out",
             3: "wait for an accumulator (tmem full) timed out", 4: "wait for a drained accumulator (tmem empty) timed out",
             5: "wait for a peer rank's flag timed out", 6: "draining in-flight copies timed out",
             7: "self-test flag wait timed out (expected in the bounded-wait test)",
             8: "a kernel's work list overflowed the space its launcher reserved"}


class KernelError(RuntimeError):
    pass


def have_cuda() -> bool:
    return torch.cuda.is_available()


def lib() -> ctypes.CDLL:
    """The loaded kernel library (built on first use when nvcc is present and no ``.so`` exists)."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.LIBPATH
                # With a compiler at hand the build is re-checked on every first use (unchanged sources cost a few hashes), so a
                # library older than the sources -- whose entry points may no longer match the Python wrappers -- is never loaded.
                # Concurrent ranks of one node serialise on a lock file.
                if _build.nvcc_path() is not None:
                    path = _locked_build()
                elif not os.path.exists(path):
                    path = _build.build()
                _lib = ctypes.CDLL(path)
                _declare(_lib)
    return _lib


def _locked_build() -> str:
    import fcntl
    os.makedirs(os.path.dirname(_build.LIBPATH), exist_ok=True)
    with open(_build.LIBPATH + ".lock", "w") as fh:
        fcntl.flock(fh, fcntl.LOCK_EX)
        try:
            return _build.build()
        finally:
            fcntl.flock(fh, fcntl.LOCK_UN)


def _declare(l: ctypes.CDLL) -> None:
    c_int, c_ll, c_f, vp = ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_void_p
    l.dttt_gemm_bf16.restype = c_int
    l.dttt_gemm_bf16.argtypes = [vp, vp, vp, c_int, c_int, c_int, c_int, c_ll, c_ll, c_ll, c_ll, c_ll, c_ll,
                                 c_int, c_int, c_int, c_int, c_f, vp, c_int, vp]
    for name, spec in _SIGNATURES.items():
        if hasattr(l, name):
            fn = getattr(l, name)
            fn.restype = spec[0]
            fn.argtypes = spec[1]


# name -> (restype, argtypes); filled by the op modules at import (see register()).
_SIGNATURES: dict[str, tuple] = {}


def register(name: str, restype, argtypes) -> None:
    _SIGNATURES[name] = (restype, argtypes)
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.restype, fn.argtypes = restype, argtypes


def status_tensor(device: torch.device | int | None = None) -> torch.Tensor:
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    t = _status.get(idx)
    if t is None:
        t = torch.zeros(4, dtype=torch.int32, device=f"cuda:{idx}")
        _status[idx] = t
    return t


def check_status(device=None, reset: bool = True) -> None:
    """Raise ``KernelError`` if a kernel on this device recorded an error since the last check."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    t = _status.get(idx)
    if t is None:
        return
    code = int(t[0].item())
    if code:
        if reset:
            t.zero_()
        raise KernelError(f"device kernel reported status {code}: {ERR_NAMES.get(code, 'unknown')}")


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


register("dttt_wait_selftest", ctypes.c_int, [ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p,
                                              ctypes.c_void_p])


def wait_selftest(flag: torch.Tensor, target: int, limit_ms: float = 2.0) -> torch.Tensor:
    """Launch the bounded-wait self-test: a kernel that waits at most ``limit_ms`` for ``flag[0] >= target`` and, when the
    wait runs out, records the self-test code in the status word (``check_status`` then raises).  Returns a one-element
    int32 tensor that receives the microseconds waited."""
    waited = torch.zeros(1, dtype=torch.int32, device=flag.device)
    st = status_tensor(flag.device)
    rc = lib().dttt_wait_selftest(ctypes.c_void_p(flag.data_ptr()), int(target), int(limit_ms * 1e6), ctypes.c_void_p(st.data_ptr()),
                                  ctypes.c_void_p(waited.data_ptr()), ctypes.c_void_p(stream_ptr()))
    if rc != 0:
        raise KernelError(f"dttt_wait_selftest launch failed rc={rc}")
    return waited
