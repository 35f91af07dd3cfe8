"""Tensor parallelism with the collective inside the GEMM kernel (sequence-parallel layout).

Between blocks an activation ``[M, H]`` is sharded by rows over the ``tp`` ranks.  A column-parallel product
(QKV, MLP gate/up, the fast-weight MLP's input side) needs all rows: ``ag_gemm`` runs ONE kernel in which four copy
warps per CTA pull the other ranks' rows over NVLink into the local gather buffer while the tcgen05 pipeline already
multiplies the rows that are here (``csrc/gemm_tcgen05.cu``, ``EPI_AG``).  A row-parallel product (attention out,
MLP down, fast-weight output) yields partial sums of all rows: ``gemm_rs`` stores every finished tile straight into
the owning rank's slot over NVLink (``EPI_RS``) and ``slot_reduce`` adds the ``tp`` slots (plus the residual).

The reference has neither tensor nor sequence parallelism (``docs/architecture.md:82``) and prevents the partitioner
from introducing one (``src/ttt/sharding.py:65-70``); this layer is new.

Ordering between ranks uses epoch flags in peer memory, never a library barrier: a kernel announces "my rows are in
place" at every peer when it starts and raises "my partials have landed" when its last CTA finishes; every wait is
bounded and reports through the status word.  A buffer is reused every second call (two buffers alternate per
shape), which together with the start-of-kernel announcement makes overwriting safe: a rank can only begin call
``k + 1`` after it finished call ``k``, and nobody pulls call ``k + 2``'s rows before everyone announced it.

``ColumnParallelLinear`` / ``RowParallelLinear`` are the autograd forms: the backward of one is the other's
collective (dX of a column-parallel layer is a GEMM -> reduce-scatter, dX of a row-parallel layer an all-gather ->
GEMM), weight gradients are local GEMMs on the gathered operand.
"""
from __future__ import annotations

import ctypes
from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from ..ops import _lib
from ..ops import gemm as _gemm
from .symm import PeerBuffer

_vp, _ll, _i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
_PP = ctypes.POINTER(_vp)
_lib.register("dttt_gemm_ag_bf16", _i, [_PP, _PP, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _ll, _i, _i, _i, _i, _i, _vp, _vp])
_lib.register("dttt_gemm_rs_bf16", _i, [_vp, _vp, _PP, _PP, _vp, _i, _i, _i, _ll, _ll, _i, _i, _i, _i, _i, _vp, _vp])
_lib.register("dttt_tp_slot_reduce", _i, [_vp, _vp, _i, _i, _ll, _vp, _vp, _vp, _vp])

BLOCK = 128


class _Gather:
    """Two alternating gather buffers ``[M, K]`` in peer memory with their ready words."""

    def __init__(self, ws: "Workspace", M: int, K: int):
        self.M, self.K = M, K
        nbytes = M * K * 2
        self.buf = [ws.region(nbytes) for _ in range(2)]
        self.ready = [torch.zeros(M // BLOCK, dtype=torch.int32, device=ws.device) for _ in range(2)]
        self.calls = 0


class _Slots:
    def __init__(self, ws: "Workspace", rows: int, N: int):
        self.rows, self.N = rows, N
        self.buf = [ws.region(ws.tp * rows * N * 2) for _ in range(2)]
        self.done = [torch.zeros(1, dtype=torch.int32, device=ws.device) for _ in range(2)]
        self.calls = 0


class Workspace:
    """Peer memory of one tensor-parallel group: a bump allocator over one ``PeerBuffer`` (identical offsets on every
    rank because every rank makes the same requests in the same order), the flag words, and the per-shape buffers."""

    def __init__(self, group, device: torch.device, nbytes: int = 1 << 30):
        self.group, self.device = group, device
        self.tp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.peer = PeerBuffer(nbytes, group, device)
        self._top = 0
        self._gathers: Dict[Tuple[int, int], _Gather] = {}
        self._slots: Dict[Tuple[int, int], _Slots] = {}
        self._flag_sets: Dict[str, Tuple[int, torch.Tensor]] = {}
        self.epoch = 0
        self.peer._bytes.zero_()
        torch.cuda.synchronize(device)
        dist.barrier(group=group)                        # every rank's flags are zero before anyone signals

    def region(self, nbytes: int) -> int:
        off = self._top
        self._top += -(-nbytes // 256) * 256
        if self._top > self.peer.nbytes:
            raise MemoryError(f"tensor-parallel workspace of {self.peer.nbytes} bytes exhausted")
        return off

    def flags(self, key: str) -> int:
        """Byte offset of a set of ``2 * tp`` flag words (one set per buffer, so epochs of different buffers never mix)."""
        if key not in self._flag_sets:
            self._flag_sets[key] = (self.region(2 * self.tp * 4), None)
        return self._flag_sets[key][0]

    def table(self, off: int):
        return self.peer.ptr_table(off)

    def view(self, off: int, shape, dtype=torch.bfloat16) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= s
        return self.peer.tensor(off, n, dtype).view(shape)

    def gather(self, M: int, K: int) -> _Gather:
        g = self._gathers.get((M, K))
        if g is None:
            g = self._gathers[(M, K)] = _Gather(self, M, K)
        return g

    def slots(self, rows: int, N: int) -> _Slots:
        s = self._slots.get((rows, N))
        if s is None:
            s = self._slots[(rows, N)] = _Slots(self, rows, N)
        return s


def _stream():
    return _vp(_lib.stream_ptr())


def ag_gemm(ws: Workspace, x_shard: torch.Tensor, w: torch.Tensor, w_is_kn: bool = True,
            out_dtype: torch.dtype = torch.bfloat16) -> Tuple[torch.Tensor, torch.Tensor]:
    """``all_gather_rows(x_shard) @ w`` in one kernel.  ``x_shard [M / tp, K]`` bf16; ``w [K, N]`` (``w_is_kn``) or
    ``[N, K]``.  Returns ``(y [M, N], x_full [M, K])``; ``x_full`` is a view of the gather buffer, valid until the
    second-next ``ag_gemm`` of the same shape."""
    rows, K = x_shard.shape
    tp, me = ws.tp, ws.rank
    M = rows * tp
    assert rows % BLOCK == 0 and x_shard.dtype == torch.bfloat16, (rows, x_shard.dtype)
    g = ws.gather(M, K)
    which = g.calls & 1
    g.calls += 1
    epoch = g.calls                                     # per-buffer-pair counter, identical on every rank
    off = g.buf[which]
    full = ws.view(off, (M, K))
    full[me * rows:(me + 1) * rows].copy_(x_shard)
    N = w.shape[1] if w_is_kn else w.shape[0]
    y = torch.empty(M, N, dtype=out_dtype, device=x_shard.device)
    wc = w if w.stride(-1) == 1 else w.contiguous()
    st = _lib.status_tensor(x_shard.device)
    foff = ws.flags(f"g{M}x{K}.{which}")
    rc = _lib.lib().dttt_gemm_ag_bf16(ws.table(off), ws.table(foff), _vp(g.ready[which].data_ptr()), _vp(wc.data_ptr()), _vp(y.data_ptr()),
                                      M, N, K, K, wc.stride(0), N, 1 if w_is_kn else 0, 1 if out_dtype == torch.float32 else 0, tp, me,
                                      epoch, _vp(st.data_ptr()), _stream())
    if rc:
        raise _lib.KernelError(f"gemm_ag launch failed rc={rc}")
    _gemm.LAUNCHES += 1
    return y, full


def gemm_rs(ws: Workspace, x: torch.Tensor, w: torch.Tensor, x_is_km: bool = False, w_is_kn: bool = True,
            residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``reduce_scatter_rows(x @ w)`` (+ ``residual``): ``x [M, K_local]`` (or ``[K_local, M]`` with ``x_is_km``), ``w [K_local, N]``
    (or ``[N, K_local]``); returns this rank's ``[M / tp, N]`` rows of the sum over ranks."""
    tp, me = ws.tp, ws.rank
    M = x.shape[1] if x_is_km else x.shape[0]
    Kl = x.shape[0] if x_is_km else x.shape[1]
    N = w.shape[1] if w_is_kn else w.shape[0]
    assert M % (BLOCK * tp) == 0 and N % 8 == 0, (M, N)
    rows = M // tp
    s = ws.slots(rows, N)
    which = s.calls & 1
    s.calls += 1
    epoch = s.calls
    off = s.buf[which]
    xc = x if x.stride(-1) == 1 else x.contiguous()
    wc = w if w.stride(-1) == 1 else w.contiguous()
    st = _lib.status_tensor(x.device)
    foff = ws.flags(f"s{rows}x{N}.{which}")
    rc = _lib.lib().dttt_gemm_rs_bf16(_vp(xc.data_ptr()), _vp(wc.data_ptr()), ws.table(off), ws.table(foff), _vp(s.done[which].data_ptr()),
                                      M, N, Kl, xc.stride(0), wc.stride(0), 1 if x_is_km else 0, 1 if w_is_kn else 0, tp, me, epoch,
                                      _vp(st.data_ptr()), _stream())
    if rc:
        raise _lib.KernelError(f"gemm_rs launch failed rc={rc}")
    out = torch.empty(rows, N, dtype=torch.bfloat16, device=x.device)
    res = residual.contiguous() if residual is not None else None
    local_flags = ws.peer.local + foff + tp * 4          # the "partials have landed" half of this rank's flag words
    rc = _lib.lib().dttt_tp_slot_reduce(_vp(ws.peer.local + off), _vp(local_flags), tp, epoch, rows * N,
                                        _vp(res.data_ptr()) if res is not None else _vp(0), _vp(out.data_ptr()), _vp(st.data_ptr()), _stream())
    if rc:
        raise _lib.KernelError(f"tp_slot_reduce launch failed rc={rc}")
    _gemm.LAUNCHES += 2
    return out


class ColumnParallelLinear(torch.autograd.Function):
    """``y [M, N / tp] = gather_rows(x_shard) @ w_cols`` with ``w_cols [K, N / tp]`` this rank's column block."""

    @staticmethod
    def forward(ctx, x_shard, w, ws):
        y, full = ag_gemm(ws, x_shard, w)
        ctx.ws = ws
        ctx.save_for_backward(full.clone(), w)
        return y

    @staticmethod
    def backward(ctx, gy):
        x_full, w = ctx.saved_tensors
        ws = ctx.ws
        gy = gy.contiguous()
        gx = gemm_rs(ws, gy, w, w_is_kn=False) if ctx.needs_input_grad[0] else None          # (gy @ w^T) reduce-scattered by rows
        gw = _gemm.gemm_raw(x_full, gy, True, False, torch.float32).to(w.dtype) if ctx.needs_input_grad[1] else None
        return gx, gw, None


class RowParallelLinear(torch.autograd.Function):
    """``y_shard [M / tp, N] = reduce_scatter_rows(x @ w_rows)`` with ``x [M, K / tp]``, ``w_rows [K / tp, N]``."""

    @staticmethod
    def forward(ctx, x, w, ws, residual=None):
        ctx.ws = ws
        ctx.has_res = residual is not None
        ctx.save_for_backward(x, w)
        return gemm_rs(ws, x, w, residual=residual)

    @staticmethod
    def backward(ctx, gy_shard):
        x, w = ctx.saved_tensors
        ws = ctx.ws
        gx, g_full = ag_gemm(ws, gy_shard.contiguous(), w, w_is_kn=False)                     # gather_rows(gy) @ w^T
        gw = _gemm.gemm_raw(x, g_full, True, False, torch.float32).to(w.dtype) if ctx.needs_input_grad[1] else None
        return (gx if ctx.needs_input_grad[0] else None), gw, None, (gy_shard if ctx.has_res else None)


def column_linear(x_shard: torch.Tensor, w: torch.Tensor, ws: Workspace) -> torch.Tensor:
    return ColumnParallelLinear.apply(x_shard, w, ws)


def row_linear(x: torch.Tensor, w: torch.Tensor, ws: Workspace, residual: Optional[torch.Tensor] = None) -> torch.Tensor:
    return RowParallelLinear.apply(x, w, ws, residual)


# ======================================================================================================================
# The model-facing form: ``tp_linear`` is what ``ops.functional.linear`` calls for a weight that carries ``w.tp``.
# Sequences, not features, are divided over the group outside the trunk GEMMs: a rank holds the residual stream,
# the fast weights and the losses of its own ``B / tp`` sequences; a column-parallel product turns ``[B / tp, ...]`` rows
# into ``[B, ..., N / tp]`` (all rows, this rank's heads / MLP columns), a row-parallel one back into ``[B / tp, ..., N]``.
class TPContext:
    """A tensor-parallel group as the ops see it: the process group, its size, this rank's index and (on GPUs) the
    peer-memory workspace of the fused kernels."""

    def __init__(self, group, size: int, index: int, device: torch.device, workspace_bytes: int = 2 << 30):
        self.group, self.size, self.index, self.device = group, size, index, device
        self.ws: Optional[Workspace] = Workspace(group, device, workspace_bytes) if device.type == "cuda" else None
        self.last_gather = None            # (key, rows, gathered copy) of the latest column-parallel gather (_gathered_product)


def _all_gather_rows(x: torch.Tensor, ctx: TPContext) -> torch.Tensor:
    parts = [torch.empty_like(x) for _ in range(ctx.size)]
    dist.all_gather(parts, x.contiguous(), group=ctx.group)
    return torch.cat(parts, 0)


def _reduce_scatter_rows(y: torch.Tensor, ctx: TPContext) -> torch.Tensor:
    y = y.contiguous()
    rows = y.shape[0] // ctx.size
    if y.is_cuda:
        out = torch.empty((rows,) + tuple(y.shape[1:]), dtype=y.dtype, device=y.device)
        dist.reduce_scatter_tensor(out, y, group=ctx.group)
        return out
    dist.all_reduce(y, group=ctx.group)                    # gloo has no reduce-scatter
    return y[ctx.index * rows:(ctx.index + 1) * rows].clone()


class _GatherRows(torch.autograd.Function):
    """All-gather of the rows over the group; its adjoint is the reduce-scatter (and the other way round), so the pair
    is differentiable to any order."""

    @staticmethod
    def forward(ctx, x, tpc):
        ctx.tpc = tpc
        return _all_gather_rows(x, tpc)

    @staticmethod
    def backward(ctx, g):
        return _ScatterRows.apply(g, ctx.tpc), None


class _ScatterRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, y, tpc):
        ctx.tpc = tpc
        return _reduce_scatter_rows(y, tpc)

    @staticmethod
    def backward(ctx, g):
        return _GatherRows.apply(g, ctx.tpc), None


def _ref_linear(x2: torch.Tensor, w: torch.Tensor, kind: str, tpc: TPContext) -> torch.Tensor:
    """The library-collective statement (NCCL / gloo + a differentiable matmul): the meaning of the fused kernels, the CPU
    path, and what a recorded backward differentiates."""
    from ..ops.functional import mm
    wc = w if w.dtype == x2.dtype else w.to(x2.dtype)
    if kind == "col":
        return mm(_GatherRows.apply(x2, tpc), wc)
    return _ScatterRows.apply(mm(x2, wc), tpc)


def _gathered_product(tpc: "TPContext", x2: torch.Tensor, w: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(gather_rows(x2) @ w, gathered rows)`` for a column-parallel weight.  Consecutive products of the SAME rows (Q, K and V
    of a layer; gate and up) gather once: the first call runs the fused all-gather GEMM and keeps a copy of the gathered rows,
    the following ones are plain GEMMs on that copy.  The rows are recognised by storage address, layout and version counter;
    the context keeps the tensor alive meanwhile, so the address cannot have been handed to another tensor."""
    key = (x2.data_ptr(), tuple(x2.shape), tuple(x2.stride()), x2._version)
    last = tpc.last_gather
    if last is not None and last[0] == key:
        return _gemm.gemm_raw(last[2], w, False, False), last[2]
    y, view = ag_gemm(tpc.ws, x2, w)
    full = view.clone()
    tpc.last_gather = (key, x2, full)
    return y, full


class _TPLinear(torch.autograd.Function):
    """Fused forward and first-order backward (``ag_gemm`` / ``gemm_rs``); a backward that is being recorded (the inner
    step under the meta-gradient) is computed from ``_ref_linear`` instead, so it can be differentiated again.  The
    first-order weight gradient goes straight into the f32 master gradient buffer when the leaf carries ``grad_target``."""

    @staticmethod
    def forward(ctx, x2, w, kind, tpc):
        ctx.kind, ctx.tpc = kind, tpc
        ctx.target = getattr(w, "grad_target", None)
        if kind == "col":
            y, full = _gathered_product(tpc, x2, w)
            ctx.save_for_backward(x2, w, full)
        else:
            y = gemm_rs(tpc.ws, x2, w)
            ctx.save_for_backward(x2, w)
        return y

    @staticmethod
    def backward(ctx, g):
        from ..ops.functional import _INNER_BACKWARD
        kind, tpc = ctx.kind, ctx.tpc
        x2, w = ctx.saved_tensors[:2]
        want_w = ctx.needs_input_grad[1] and not _INNER_BACKWARD[0]
        if torch.is_grad_enabled():
            with torch.enable_grad():
                xi = x2 if x2.requires_grad else x2.detach().requires_grad_(ctx.needs_input_grad[0])
                wi = w if w.requires_grad else w.detach().requires_grad_(want_w)
                out = _ref_linear(xi, wi, kind, tpc)
                wrt = [t for t, nd in ((xi, ctx.needs_input_grad[0]), (wi, want_w)) if nd]
                grads = list(torch.autograd.grad(out, wrt, g, create_graph=True, allow_unused=True))
            gx = grads.pop(0) if ctx.needs_input_grad[0] else None
            gw = grads.pop(0) if want_w else None
            return gx, gw, None, None
        g = (g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)).contiguous()
        gx = gw = None
        if kind == "col":
            x_full = ctx.saved_tensors[2]
            if ctx.needs_input_grad[0]:
                gx = gemm_rs(tpc.ws, g, w, w_is_kn=False)                          # (g @ w^T), reduce-scattered by rows
            a_full, g_full = x_full, g
        else:
            gx_full, g_full = ag_gemm(tpc.ws, g, w, w_is_kn=False)                 # gather_rows(g) @ w^T
            gx = gx_full if ctx.needs_input_grad[0] else None
            a_full = x2
        if want_w:
            if ctx.target is not None:
                gbuf, layer = ctx.target
                _gemm.gemm_raw(a_full, g_full, True, False, torch.float32, out=gbuf if layer is None else gbuf[layer], accumulate=True)
            else:
                gw = _gemm.gemm_raw(a_full, g_full, True, False)
        return gx, gw, None, None


def tp_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w`` for a tensor-parallel weight leaf (``w.tp = (kind, TPContext)``).  ``kind == "col"``: ``x [B / tp, ..., K]`` ->
    ``[B, ..., N / tp]`` (+ this rank's slice of the bias); ``"row"``: ``x [B, ..., K / tp]`` -> ``[B / tp, ..., N]``."""
    from ..ops.functional import use_kernels
    kind, tpc = w.tp
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    rows = x2.shape[0]
    fused = (tpc.ws is not None and use_kernels(x2) and w.dtype == torch.bfloat16
             and (rows % BLOCK == 0 if kind == "col" else rows % (BLOCK * tpc.size) == 0))
    if fused and (torch.is_grad_enabled() and (x2.requires_grad or w.requires_grad)):
        y2 = _TPLinear.apply(x2, w, kind, tpc)
    elif fused:
        y2 = _gathered_product(tpc, x2, w)[0] if kind == "col" else gemm_rs(tpc.ws, x2, w)
    else:
        y2 = _ref_linear(x2, w, kind, tpc)
    if kind == "col":
        y = y2.view(lead[0] * tpc.size, *lead[1:], w.shape[-1])
    else:
        if lead[0] % tpc.size:
            raise ValueError(f"row-parallel product: {lead[0]} sequences do not divide over {tpc.size} ranks")
        y = y2.view(lead[0] // tpc.size, *lead[1:], w.shape[-1])
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y
