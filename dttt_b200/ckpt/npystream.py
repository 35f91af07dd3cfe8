"""A checkpoint file is a byte stream of ``.npy`` records split into parts of at most 4 GiB.

This is the byte format the reference writes (``eqx.tree_serialise_leaves`` into its ``ShardedFileWriter``,
``src/ttt/checkpoint.py:103-110``, ``src/ttt/sharded_io.py:6-46``): one ``numpy.save`` record per array leaf,
in pytree-flatten order, the concatenation cut into ``<base>.part000, .part001, ...``.  A single unsplit file
named ``<base>`` is accepted on reading (``sharded_io.py:84-229``).  Records are written and parsed one at a
time, so neither side ever holds more than one array.
"""
from __future__ import annotations

import glob
import os
from typing import Iterable, Iterator, List, Optional

import numpy as np

PART_BYTES = 4 * 1024 ** 3


class PartWriter:
    """Write-only binary stream over ``<base>.partNNN`` files."""

    def __init__(self, base: str, max_bytes: int = PART_BYTES):
        self.base, self.max_bytes = base, max_bytes
        self._idx, self._in_part, self._total = 0, 0, 0
        os.makedirs(os.path.dirname(os.path.abspath(base)), exist_ok=True)
        self._fh = open(self._name(0), "wb")

    def _name(self, i: int) -> str:
        return f"{self.base}.part{i:03d}"

    def write(self, data) -> int:
        view = memoryview(data).cast("B")
        pos, n = 0, len(view)
        while pos < n:
            room = self.max_bytes - self._in_part
            if room <= 0:
                self._fh.close()
                self._idx += 1
                self._fh, self._in_part = open(self._name(self._idx), "wb"), 0
                room = self.max_bytes
            take = min(room, n - pos)
            self._fh.write(view[pos:pos + take])
            pos, self._in_part, self._total = pos + take, self._in_part + take, self._total + take
        return n

    def tell(self) -> int:
        return self._total

    def flush(self) -> None:
        self._fh.flush()

    def close(self) -> None:
        if self._fh is not None:
            self._fh.close()
            self._fh = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class PartReader:
    """Read-only binary stream over the parts of ``base`` (or the single file ``base``)."""

    def __init__(self, base: str):
        if os.path.exists(base + ".part000"):
            self.files = sorted(glob.glob(base + ".part*"))
            for i, f in enumerate(self.files):
                suffix = f.rsplit(".part", 1)[-1]
                if not suffix.isdigit() or int(suffix) != i:
                    raise ValueError(f"checkpoint parts of {base} are not contiguous: expected part{i:03d}, found {os.path.basename(f)}")
        elif os.path.exists(base):
            self.files = [base]
        else:
            raise FileNotFoundError(base)
        self.sizes = [os.path.getsize(f) for f in self.files]
        self.total = sum(self.sizes)
        self._pos, self._cur, self._fh = 0, -1, None

    def _open_at(self, pos: int):
        acc = 0
        for i, sz in enumerate(self.sizes):
            if pos < acc + sz or i == len(self.sizes) - 1:
                if i != self._cur:
                    if self._fh:
                        self._fh.close()
                    self._fh, self._cur = open(self.files[i], "rb"), i
                self._fh.seek(pos - acc)
                return acc + sz - pos
            acc += sz
        return 0

    def read(self, n: int = -1) -> bytes:
        if n < 0:
            n = self.total - self._pos
        out = bytearray()
        while n > 0 and self._pos < self.total:
            room = self._open_at(self._pos)
            chunk = self._fh.read(min(n, room))
            if not chunk:
                break
            out += chunk
            self._pos += len(chunk)
            n -= len(chunk)
        return bytes(out)

    def readinto(self, buf) -> int:
        data = self.read(len(buf))
        buf[:len(data)] = data
        return len(data)

    def tell(self) -> int:
        return self._pos

    def seek(self, offset: int, whence: int = 0) -> int:
        self._pos = max(0, min(self.total, {0: offset, 1: self._pos + offset, 2: self.total + offset}[whence]))
        return self._pos

    def close(self) -> None:
        if self._fh:
            self._fh.close()
            self._fh = None

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


def write_records(base: str, arrays: Iterable[np.ndarray], max_bytes: int = PART_BYTES) -> int:
    """Write one ``.npy`` record per array; returns the number of records."""
    n = 0
    with PartWriter(base, max_bytes) as w:
        for a in arrays:
            a = np.asarray(a)
            np.lib.format.write_array(w, a if a.flags.c_contiguous else np.ascontiguousarray(a), allow_pickle=False)
            n += 1
    return n


def read_records(base: str) -> Iterator[np.ndarray]:
    """Yield the arrays of a record stream in order."""
    with PartReader(base) as r:
        while r.tell() < r.total:
            yield np.lib.format.read_array(r, allow_pickle=False)
