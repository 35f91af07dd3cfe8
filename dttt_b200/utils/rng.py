"""Counter-based random numbers with the keying structure of the reference's JAX PRNG.

The reference draws every mask from stateless keys: ``PRNGKey(seed)`` folded with the step, split
into (unused, outer-mask, inner) keys, the inner key split per chunk and sequence, and so on
(``src/ttt/chunk_scan.py:229-237``, ``src/ttt/train.py:1123-1126``).  Bitwise resume and the
"batch-shape independent" row-wise evaluation keys rest on that structure, so it is reproduced here
with the same generator, Threefry-2x32 (20 rounds), and the same derivations JAX uses when
``jax_threefry_partitionable`` is on (the default of the reference's JAX version):

* ``key(seed)``            -> ``(hi32(seed), lo32(seed))``
* ``split(key, n)``        -> ``threefry(key, counter = (0, i))`` for ``i < n``, both output words
* ``fold_in(key, d)``      -> ``threefry(key, counter = (0, d))``
* ``bits(key, shape)``     -> ``w0 ^ w1`` of ``threefry(key, counter = (hi(i), lo(i)))`` over the flat index
* ``uniform``              -> ``bitcast((bits >> 9) | 0x3f800000) - 1``

Everything is implemented with int64 torch ops masked to 32 bits, so the same code runs on CPU and
on the GPU, vectorised over any leading "key batch" shape.  Keys are int64 tensors ``[..., 2]``.
"""
from __future__ import annotations

import math
from typing import Sequence, Tuple

import torch

M32 = 0xFFFFFFFF
_ROT = ((13, 15, 26, 6), (17, 29, 16, 24))


def _rotl(x: torch.Tensor, r: int) -> torch.Tensor:
    return ((x << r) | (x >> (32 - r))) & M32


def threefry2x32(k0: torch.Tensor, k1: torch.Tensor, x0: torch.Tensor, x1: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Threefry-2x32 with 20 rounds; all arguments int64 tensors holding 32-bit values (broadcastable)."""
    ks = (k0, k1, (k0 ^ k1 ^ 0x1BD11BDA) & M32)
    x0 = (x0 + ks[0]) & M32
    x1 = (x1 + ks[1]) & M32
    for i in range(5):
        for r in _ROT[i % 2]:
            x0 = (x0 + x1) & M32
            x1 = _rotl(x1, r) ^ x0
        x0 = (x0 + ks[(i + 1) % 3]) & M32
        x1 = (x1 + ks[(i + 2) % 3] + (i + 1)) & M32
    return x0, x1


def key(seed: int, device=None) -> torch.Tensor:
    seed = int(seed) & 0xFFFFFFFFFFFFFFFF
    return torch.tensor([(seed >> 32) & M32, seed & M32], dtype=torch.int64, device=device)


def _iota(n: int, device) -> Tuple[torch.Tensor, torch.Tensor]:
    i = torch.arange(n, dtype=torch.int64, device=device)
    return (i >> 32) & M32, i & M32


def split(k: torch.Tensor, n: int = 2) -> torch.Tensor:
    """``k [..., 2]`` -> ``[..., n, 2]``."""
    hi, lo = _iota(n, k.device)
    y0, y1 = threefry2x32(k[..., 0:1], k[..., 1:2], hi, lo)
    return torch.stack([y0, y1], dim=-1)


def fold_in(k: torch.Tensor, data) -> torch.Tensor:
    """``k [..., 2]`` folded with an integer (python int or tensor broadcastable to the key batch)."""
    d = torch.as_tensor(data, dtype=torch.int64, device=k.device) & M32
    y0, y1 = threefry2x32(k[..., 0], k[..., 1], torch.zeros_like(d), d)
    return torch.stack([y0, y1], dim=-1)


_CHUNK = 1 << 24       # elements generated at a time (bounds the int64 temporaries)


def bits(k: torch.Tensor, shape: Sequence[int], start: int = 0, count: int = -1) -> torch.Tensor:
    """32 random bits per element: ``k [..., 2]`` -> int64 ``[..., *shape]`` (or the flat slice
    ``[start, start+count)`` of it when ``count >= 0``)."""
    n = int(math.prod(shape)) if len(shape) else 1
    lo_i, hi_i = (0, n) if count < 0 else (start, start + count)
    i = torch.arange(lo_i, hi_i, dtype=torch.int64, device=k.device)
    y0, y1 = threefry2x32(k[..., 0:1], k[..., 1:2], (i >> 32) & M32, i & M32)
    out = y0 ^ y1
    return out.reshape(tuple(k.shape[:-1]) + tuple(shape)) if count < 0 else out


def _to_unit(b: torch.Tensor) -> torch.Tensor:
    return ((b >> 9) | 0x3F800000).to(torch.int32).view(torch.float32) - 1.0


def uniform(k: torch.Tensor, shape: Sequence[int] = (), lo: float = 0.0, hi: float = 1.0) -> torch.Tensor:
    """float32 uniform on ``[lo, hi)``; ``k [..., 2]`` -> ``[..., *shape]``."""
    n = int(math.prod(shape)) if len(shape) else 1
    if k.is_cuda and n * max(1, k.numel() // 2) >= 1024 and k.numel() // 2 <= 65535:
        # bulk draws on a GPU: one launch of the counter-RNG kernel (same bits as the statement below)
        from ..ops import kernels
        if kernels.available("mask_rng"):
            u = kernels.threefry_uniform(k.reshape(-1, 2), n).reshape(tuple(k.shape[:-1]) + tuple(shape))
            if lo != 0.0 or hi != 1.0:
                u = torch.clamp_min(u * (hi - lo) + lo, lo)
            return u
    if n <= _CHUNK or k.dim() > 1:
        u = _to_unit(bits(k, shape))
    else:
        u = torch.cat([_to_unit(bits(k, shape, s, min(_CHUNK, n - s))) for s in range(0, n, _CHUNK)]).reshape(*shape)
    if lo != 0.0 or hi != 1.0:
        u = torch.clamp_min(u * (hi - lo) + lo, lo)
    return u


def normal(k: torch.Tensor, shape: Sequence[int]) -> torch.Tensor:
    """float32 standard normal by the inverse error function of a uniform on (-1, 1)."""
    lo = float(torch.nextafter(torch.tensor(-1.0), torch.tensor(0.0)))
    u = uniform(k, shape, lo, 1.0)
    return math.sqrt(2.0) * torch.erfinv(u)


def bernoulli(k: torch.Tensor, p, shape: Sequence[int]) -> torch.Tensor:
    return uniform(k, shape) < p
