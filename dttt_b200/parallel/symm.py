"""Peer-accessible device buffers over CUDA IPC: the memory the fused compute+collective kernels address.

``PeerBuffer(nbytes, group)`` allocates ``nbytes`` on this rank's GPU, exchanges IPC handles over the process
group and opens every peer's allocation, so ``ptrs[r]`` is a device pointer, valid on THIS GPU, to rank ``r``'s
buffer (``ptrs[self]`` is the local allocation).  Loads and stores through a peer pointer travel over NVLink /
NVSwitch.  ``tensor(...)`` views the local allocation as a torch tensor; ``ptr_table(offset)`` is a ctypes array
of the peers' pointers at a byte offset, the argument the kernels in ``csrc/comm_fused.cu`` take.

The reference has no counterpart: its collectives are inserted by the XLA partitioner (``src/ttt/sharding.py``);
this is the explicit NVLink layer that replaces them on the optimiser-step path.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch
import torch.distributed as dist

from ..ops import _lib

_vp, _ll, _i, _f = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int, ctypes.c_float
_lib.register("dttt_peer_alloc", _i, [ctypes.POINTER(_vp), _ll])
_lib.register("dttt_peer_free", _i, [_vp])
_lib.register("dttt_peer_export", _i, [_vp, _vp])
_lib.register("dttt_peer_open", _i, [_vp, ctypes.POINTER(_vp)])
_lib.register("dttt_peer_close", _i, [_vp])
_lib.register("dttt_ipc_handle_bytes", _i, [])
_lib.register("dttt_reduce_scatter_sumsq", _i, [ctypes.POINTER(_vp), _i, _i, _ll, _ll, _f, _vp, _vp, _vp])
_lib.register("dttt_adamw_allgather", _i, [_vp, _vp, _vp, _vp, _ll, _f, _f, _f, _f, _f, _f, _f, _f, ctypes.POINTER(_vp), _i, _i, _ll, _i, _vp])


class _Raw:
    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerBuffer:
    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.nbytes = int(-(-nbytes // 256) * 256)
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        lib = _lib.lib()
        p = _vp()
        rc = lib.dttt_peer_alloc(ctypes.byref(p), self.nbytes)
        if rc:
            raise _lib.KernelError(f"peer buffer allocation of {self.nbytes} bytes failed (cuda error {rc})")
        self.local = p.value
        self.ptrs: List[int] = [0] * self.world
        self.ptrs[self.rank] = self.local
        self._opened: List[int] = []
        if self.world > 1:
            hb = lib.dttt_ipc_handle_bytes()
            buf = (ctypes.c_ubyte * hb)()
            rc = lib.dttt_peer_export(_vp(self.local), ctypes.cast(buf, _vp))
            if rc:
                raise _lib.KernelError(f"cudaIpcGetMemHandle failed (cuda error {rc})")
            handles: List[Optional[bytes]] = [None] * self.world
            dist.all_gather_object(handles, bytes(buf), group=group)
            for r, h in enumerate(handles):
                if r == self.rank:
                    continue
                src = (ctypes.c_ubyte * hb).from_buffer_copy(h)
                q = _vp()
                rc = lib.dttt_peer_open(ctypes.cast(src, _vp), ctypes.byref(q))
                if rc:
                    raise _lib.KernelError(f"cudaIpcOpenMemHandle for rank {r} failed (cuda error {rc})")
                self.ptrs[r] = q.value
                self._opened.append(q.value)
        self._bytes = torch.as_tensor(_Raw(self.local, self.nbytes), device=self.device)

    def tensor(self, byte_offset: int, numel: int, dtype: torch.dtype) -> torch.Tensor:
        size = numel * torch.empty(0, dtype=dtype).element_size()
        return self._bytes[byte_offset:byte_offset + size].view(dtype)

    def ptr_table(self, byte_offset: int = 0):
        return (_vp * self.world)(*[_vp(p + byte_offset) for p in self.ptrs])

    def close(self) -> None:
        lib = _lib.lib()
        for q in self._opened:
            lib.dttt_peer_close(_vp(q))
        self._opened = []
        if self.local:
            self._bytes = None
            lib.dttt_peer_free(_vp(self.local))
            self.local = 0


def reduce_scatter_sumsq(table, world: int, self_rank: int, off: int, n: int, scale: float, out: torch.Tensor, sumsq: torch.Tensor) -> None:
    rc = _lib.lib().dttt_reduce_scatter_sumsq(table, world, self_rank, off, n, float(scale), _vp(out.data_ptr()), _vp(sumsq.data_ptr()),
                                              _vp(_lib.stream_ptr()))
    if rc:
        raise _lib.KernelError(f"reduce_scatter_sumsq launch failed rc={rc}")


def adamw_allgather(p, m, v, g, lr, b1, b2, eps, wd, bc1, bc2, gscale, table, world: int, self_rank: int, off: int, lo_is_bf16: bool) -> None:
    rc = _lib.lib().dttt_adamw_allgather(_vp(p.data_ptr()), _vp(m.data_ptr()), _vp(v.data_ptr()), _vp(g.data_ptr()), p.numel(), float(lr),
                                         float(b1), float(b2), float(eps), float(wd), float(bc1), float(bc2), float(gscale), table, world,
                                         self_rank, off, 1 if lo_is_bf16 else 0, _vp(_lib.stream_ptr()))
    if rc:
        raise _lib.KernelError(f"adamw_allgather launch failed rc={rc}")
