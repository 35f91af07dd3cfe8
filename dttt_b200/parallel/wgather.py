"""FSDP weight all-gather fused into the consuming GEMM (``csrc/gemm_tcgen05.cu``, epilogue mode 5).

The reference shards every array over the FSDP axis and lets the partitioner all-gather one layer's weights per use
(``src/ttt/model.py:580-586``, ``src/ttt/sharding.py:39-52``, ``src/ttt/train.py:678-707``).  Here the option
``TrainConfig.shard_compute`` does the same for the prefix layers' matrices without a collective launch: after the
optimiser step a rank refreshes only ITS slice of the flat bf16 parameter space (the slice of its f32 master), and every
product ``x @ w`` (and ``g @ w^T`` in the backward) pulls the weight from the owners' slices inside the GEMM kernel -
four copy warps per CTA, 64 weight rows at a time, peer loads over NVLink into a dense local staging buffer that the TMA
producer reads as soon as the rows a tile needs are marked ready.  Nothing outside a rank's own slice is ever read from
its own compute buffer, so that part of the buffer carries no state between steps.

Ordering: the shards are final before any rank's forward starts (the optimiser step ends with a group barrier) and do
not change until every rank's backward has finished (the gradient reduce-scatter starts with one).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from ..ops import _lib

_vp, _ll, _i = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
_PP = ctypes.POINTER(_vp)
_lib.register("dttt_gemm_wg_bf16", _i, [_vp, _PP, _vp, _vp, _vp, _vp, _i, _i, _i, _ll, _ll, _i, _ll, _ll, _i, _i, _i, _i, _i, _i, _vp, _vp])

ROW_BLOCK = 64          # weight rows per copy block / ready word (WG_ROWS in the kernel)
LAUNCHES = 0


class WeightGather:
    """What the fused kernel needs to find a flat-sharded weight: the ranks' shard pointers, the shard length, a staging
    buffer for one whole weight and the ready words (one per 64 rows; their epoch grows with every launch)."""

    def __init__(self, shard_table, shard_elems: int, world: int, rank: int, device: torch.device, max_weight_elems: int,
                 max_rows: int):
        self.table, self.shard_elems, self.world, self.rank, self.device = shard_table, int(shard_elems), world, rank, device
        self.stage = torch.empty(max_weight_elems, dtype=torch.bfloat16, device=device)
        self.ready = torch.zeros(-(-max_rows // ROW_BLOCK) + 8, dtype=torch.int32, device=device)
        self.count = torch.zeros_like(self.ready)       # parts of a block copied so far (the kernel leaves it at zero)
        self.epoch = 0

    def gemm(self, a: torch.Tensor, w_shape, flat_off: int, transpose_w: bool, out_dtype=torch.bfloat16,
             out: Optional[torch.Tensor] = None, accumulate: bool = False, max_ctas: int = 0) -> torch.Tensor:
        """``a [M, K] @ W`` (``transpose_w`` False, ``W [K, N]``) or ``a [M, N'] @ W^T`` (True, ``W [K', N']``) where ``W`` is the
        weight of shape ``w_shape`` whose first element has index ``flat_off`` in the sharded flat space."""
        rows, cols = int(w_shape[0]), int(w_shape[1])
        assert a.dim() == 2 and a.dtype == torch.bfloat16 and a.is_cuda and a.stride(1) == 1
        M = a.shape[0]
        if transpose_w:
            assert a.shape[1] == cols, (tuple(a.shape), w_shape)
            N, K, on_k = rows, cols, 0                    # weight rows are the output columns
        else:
            assert a.shape[1] == rows, (tuple(a.shape), w_shape)
            N, K, on_k = cols, rows, 1                    # weight rows are the contraction index
        assert rows * cols <= self.stage.numel() and rows <= (self.ready.numel() - 8) * ROW_BLOCK
        if out is None:
            out = torch.empty(M, N, dtype=out_dtype, device=a.device)
        assert out.dtype in (torch.bfloat16, torch.float32) and out.stride(1) == 1
        self.epoch += 1
        st = _lib.status_tensor(a.device)
        rc = _lib.lib().dttt_gemm_wg_bf16(_vp(a.data_ptr()), self.table, _vp(self.stage.data_ptr()), _vp(self.ready.data_ptr()),
                                          _vp(self.count.data_ptr()), _vp(out.data_ptr()), M, N, K, a.stride(0), out.stride(0), on_k, int(flat_off), self.shard_elems,
                                          self.world, self.rank, self.epoch, 1 if out.dtype == torch.float32 else 0,
                                          1 if accumulate else 0, int(max_ctas), _vp(st.data_ptr()),
                                          _vp(torch.cuda.current_stream().cuda_stream))
        if rc:
            raise _lib.KernelError(f"gemm_wg launch failed rc={rc} (M={M} N={N} K={K} on_k={on_k})")
        global LAUNCHES
        LAUNCHES += 1
        return out

    def supports(self, w_shape) -> bool:
        rows, cols = int(w_shape[0]), int(w_shape[1])
        return rows % ROW_BLOCK == 0 and cols % 8 == 0 and rows * cols <= self.stage.numel()


class _WGLinear(torch.autograd.Function):
    """``x @ w`` for a weight leaf that carries ``w.wg = (WeightGather, flat offset)``: the forward and the input gradient
    gather the weight inside their GEMMs; the weight gradient ``x^T g`` is added to the leaf's f32 gradient buffer by the
    plain GEMM's epilogue (it does not need the weight)."""

    @staticmethod
    def forward(ctx, x, w):
        wg, off = w.wg
        ctx.save_for_backward(x)
        ctx.w = w
        return wg.gemm(x, w.shape, off, False)

    @staticmethod
    def backward(ctx, g):
        from ..ops import gemm as _gemm
        from ..ops.functional import _INNER_BACKWARD
        if torch.is_grad_enabled():
            raise RuntimeError("a sharded-compute weight is used by the prefix layers only, whose backward is never recorded")
        (x,), w = ctx.saved_tensors, ctx.w
        wg, off = w.wg
        g = g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)
        g = g if g.stride(1) == 1 else g.contiguous()
        gx = gw = None
        if ctx.needs_input_grad[0]:
            gx = wg.gemm(g, w.shape, off, True)
        if ctx.needs_input_grad[1] and not _INNER_BACKWARD[0]:
            target = getattr(w, "grad_target", None)
            if target is not None:
                gbuf, layer = target
                _gemm.gemm_raw(x, g, True, False, torch.float32, out=gbuf if layer is None else gbuf[layer], accumulate=True)
            else:
                gw = _gemm.gemm_raw(x, g, True, False)
        return gx, gw


def wg_linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w (+ bias)`` through the gather-fused GEMM; called by ``ops.functional.linear`` for leaves that carry ``w.wg``."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    x2 = x2 if x2.dtype == torch.bfloat16 else x2.to(torch.bfloat16)
    x2 = x2 if x2.stride(1) == 1 and x2.stride(0) % 8 == 0 else x2.contiguous()
    if torch.is_grad_enabled() and (x2.requires_grad or w.requires_grad):
        y = _WGLinear.apply(x2, w)
    else:
        wg, off = w.wg
        y = wg.gemm(x2, w.shape, off, False)
    y = y.view(*lead, w.shape[-1])
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y
