"""Python front ends of the hand-written CUDA kernels other than the GEMM (``ops.gemm``).

``available(name)`` says whether the named kernel family is compiled into the loaded library; the
dispatchers in ``ops.functional`` ask before using one.  Families are added to ``_FAMILIES`` by the
sections below as their symbols are found.
"""
from __future__ import annotations

import ctypes
from typing import Dict

import torch

from . import _lib

_FAMILIES: Dict[str, bool] = {}
_DISABLED = set()
LAUNCHES = 0


def available(name: str) -> bool:
    if name in _DISABLED or not torch.cuda.is_available():
        return False
    ok = _FAMILIES.get(name)
    if ok is None:
        sym = _SYMBOL.get(name)
        ok = bool(sym) and hasattr(_lib.lib(), sym)
        _FAMILIES[name] = ok
    return ok


def disable(name: str) -> None:
    _DISABLED.add(name)


def enable(name: str) -> None:
    _DISABLED.discard(name)


# family -> a symbol whose presence means the family is built
_SYMBOL: Dict[str, str] = {}
