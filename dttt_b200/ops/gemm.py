"""Matrix products on the tcgen05 GEMM kernel (``csrc/gemm_tcgen05.cu``), differentiable to any order.

``mm(a, b, ta, tb)`` computes ``op(a) @ op(b)`` for 2-D or batched 3-D operands.  On a CUDA device
with bf16 operands the product runs on the hand-written kernel for every transposition (the kernel
reads K-major and MN-major tiles alike, so no operand is ever transposed in memory); elsewhere
(CPU, f32 test configurations) it is ``torch.matmul``.  The backward of a product is two more
products issued through the same differentiable entry point, so the meta-gradient (the outer
gradient through the inner step, reference src/ttt/chunk_scan.py:604-625) differentiates it again
without special code.

Weights follow the reference layout ``[in, out]`` applied as ``x @ w`` (reference
src/ttt/model.py:137-148).
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _lib

import os

_FORCE_TORCH = False          # tests flip this to compare the kernel against torch.matmul
LAUNCHES = 0                  # kernel launches issued by this module (bench accounting)
# DTTT_EMULATE=1: run the kernel code paths (custom autograd functions, in-place f32 gradient accumulation,
# staged backward) on CPU bf16 tensors with every device kernel replaced by its PyTorch statement.  It lets the
# CPU test-suite exercise exactly the control flow a GPU run takes.
EMULATE = os.environ.get("DTTT_EMULATE", "0") == "1"
# Products of at least PAIR_MIN rows and PAIR_MIN_N columns that do not accumulate into their output run on CTA pairs
# (tcgen05 cta_group::2): +12-17 % on the model's large shapes, +5-8 % at 2048 rows; narrower outputs and the long-K
# accumulating weight gradients (which take the 256 x 256 single-CTA form) measured faster on one CTA.  DTTT_GEMM_PAIR=0 turns
# the pairs off.
PAIR = os.environ.get("DTTT_GEMM_PAIR", "1") == "1"
SHAPE_LOG = None        # a dict while a profile wants the launches counted by problem shape (tools/step_profile.py)
PAIR_MIN = 256
PAIR_MIN_N = 1024
PAIR_ACCUMULATE = os.environ.get("DTTT_GEMM_PAIR_ACC", "0") == "1"     # CTA pairs also for C += products (weight gradients)
PAIR_MIN_TILES = 100    # below about 100 pair tiles (74 pairs of SMs) one CTA per 128-wide tile fills the machine better
_lib.register("dttt_gemm_pair_bf16", ctypes.c_int, [ctypes.c_void_p] * 3 + [ctypes.c_int] * 4 + [ctypes.c_longlong] * 6 + [ctypes.c_int] * 4
              + [ctypes.c_float, ctypes.c_void_p, ctypes.c_void_p])


def _kernel_ok(x: torch.Tensor) -> bool:
    return (x.is_cuda or EMULATE) and x.dtype == torch.bfloat16 and not _FORCE_TORCH


def _emulated_gemm(a, b, ta, tb, out_dtype, out, accumulate, alpha):
    x = a.transpose(-1, -2) if ta else a
    y = b.transpose(-1, -2) if tb else b
    r = torch.matmul(x.float(), y.float()) * alpha
    if out is None:
        return r.to(out_dtype)
    if accumulate:
        out.copy_((out.float() + r).to(out.dtype))
    else:
        out.copy_(r.to(out.dtype))
    return out


def _as_rows(x: torch.Tensor) -> torch.Tensor:
    """A view (or copy) whose last dim is contiguous, whose row/batch strides are multiples of 8
    elements and whose base is 16-byte aligned: what a tensor map accepts."""
    ok = x.stride(-1) == 1 and x.stride(-2) % 8 == 0 and x.data_ptr() % 16 == 0
    if x.dim() == 3:
        ok = ok and (x.stride(0) % 8 == 0 or x.shape[0] == 1)
        # rows of one batch entry must not alias rows of the next in a way a 3-D map cannot express
        ok = ok and x.stride(-2) >= x.shape[-1]
    return x if ok else x.contiguous()


def gemm_raw(a: torch.Tensor, b: torch.Tensor, ta: bool, tb: bool, out_dtype: torch.dtype = torch.bfloat16,
             out: Optional[torch.Tensor] = None, accumulate: bool = False, alpha: float = 1.0,
             max_ctas: int = 0) -> torch.Tensor:
    """One kernel launch, no autograd.  ``a``: ``[.., M, K]`` (``[.., K, M]`` with ``ta``), ``b``:
    ``[.., K, N]`` (``[.., N, K]`` with ``tb``); 2-D or 3-D with equal batch; a 2-D operand is shared by
    every batch entry of a 3-D one.  ``out`` (+ ``accumulate``) writes / adds into an existing tensor."""
    global LAUNCHES
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, (a.dtype, b.dtype)
    if not a.is_cuda:
        LAUNCHES += 1
        return _emulated_gemm(a, b, ta, tb, out_dtype, out, accumulate, alpha)
    a, b = _as_rows(a), _as_rows(b)
    M, K = (a.shape[-1], a.shape[-2]) if ta else (a.shape[-2], a.shape[-1])
    Kb, N = (b.shape[-1], b.shape[-2]) if tb else (b.shape[-2], b.shape[-1])
    assert K == Kb, f"contraction mismatch {tuple(a.shape)} ta={ta} x {tuple(b.shape)} tb={tb}"
    batch = 1
    if a.dim() == 3 or b.dim() == 3:
        batch = a.shape[0] if a.dim() == 3 else b.shape[0]
        if a.dim() == 3 and b.dim() == 3:
            assert a.shape[0] == b.shape[0]
    a_batch = a.stride(0) if a.dim() == 3 else 0
    b_batch = b.stride(0) if b.dim() == 3 else 0
    if batch > 1 and a.dim() == 3 and b.dim() == 2 and not ta and a.is_contiguous():
        # shared right operand: fold the batch into the rows
        res = gemm_raw(a.reshape(-1, a.shape[-1]), b, False, tb, out_dtype,
                       None if out is None else out.view(-1, out.shape[-1]), accumulate, alpha, max_ctas)
        return res.view(batch, M, N)
    if batch > 1 and (a_batch == 0 or b_batch == 0):
        # a shared 2-D operand with a batched partner: a zero batch stride is a legal tensor-map stride
        # only as an explicit expand; materialise the small side.
        if a.dim() == 2:
            a = a.unsqueeze(0).expand(batch, -1, -1).contiguous(); a_batch = a.stride(0)
        if b.dim() == 2:
            b = b.unsqueeze(0).expand(batch, -1, -1).contiguous(); b_batch = b.stride(0)
    shape = (M, N) if batch == 1 and a.dim() == 2 and b.dim() == 2 else (batch, M, N)
    if out is None:
        assert not accumulate
        out = torch.empty(shape, dtype=out_dtype, device=a.device)
    else:
        assert out.shape == torch.Size(shape) and out.stride(-1) == 1, (out.shape, shape)
    c_batch = out.stride(0) if out.dim() == 3 else 0
    st = _lib.status_tensor(a.device)
    if SHAPE_LOG is not None:
        key = (M, N, K, batch, int(ta), int(tb), int(accumulate))
        SHAPE_LOG[key] = SHAPE_LOG.get(key, 0) + 1
    if (PAIR and max_ctas == 0 and M >= PAIR_MIN and N >= PAIR_MIN_N and (PAIR_ACCUMULATE or not accumulate)
            and -(-M // 256) * -(-N // 256) * batch >= PAIR_MIN_TILES):
        # CTA pairs (csrc/gemm_pair_tcgen05.cu): each CTA of a cluster loads half of B, one instruction covers 256 x 256
        rc = _lib.lib().dttt_gemm_pair_bf16(
            ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(out.data_ptr()),
            M, N, K, batch, a.stride(-2), b.stride(-2), out.stride(-2), a_batch, b_batch, c_batch,
            1 if ta else 0, 0 if tb else 1, 1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
            float(alpha), ctypes.c_void_p(st.data_ptr()), ctypes.c_void_p(_lib.stream_ptr()))
        if rc != 0:
            raise _lib.KernelError(f"dttt_gemm_pair_bf16 launch failed rc={rc} for M={M} N={N} K={K} batch={batch} ta={ta} tb={tb}")
        LAUNCHES += 1
        return out
    rc = _lib.lib().dttt_gemm_bf16(
        ctypes.c_void_p(a.data_ptr()), ctypes.c_void_p(b.data_ptr()), ctypes.c_void_p(out.data_ptr()),
        M, N, K, batch, a.stride(-2), b.stride(-2), out.stride(-2), a_batch, b_batch, c_batch,
        1 if ta else 0, 0 if tb else 1, 1 if out.dtype == torch.float32 else 0, 1 if accumulate else 0,
        float(alpha), ctypes.c_void_p(st.data_ptr()), max_ctas, ctypes.c_void_p(_lib.stream_ptr()))
    if rc != 0:
        raise _lib.KernelError(f"dttt_gemm_bf16 launch failed rc={rc} for M={M} N={N} K={K} batch={batch} "
                               f"ta={ta} tb={tb}")
    LAUNCHES += 1
    return out


def set_tile_form(mode: int) -> None:
    """Tile form of the plain GEMM when N > 128: ``-1`` chosen per shape (the default), ``0`` always 128 x 256 tiles with
    double-buffered accumulators, ``1`` 256 x 256 tiles (two row halves sharing every B tile) wherever legal."""
    from ctypes import c_int
    l = _lib.lib()
    l.dttt_gemm_tile256.argtypes = [c_int]
    l.dttt_gemm_tile256.restype = None
    l.dttt_gemm_tile256(int(mode))


def _torch_mm(a, b, ta, tb, out_dtype):
    x = a.transpose(-1, -2) if ta else a
    y = b.transpose(-1, -2) if tb else b
    if out_dtype is not None and out_dtype != x.dtype and x.dtype == torch.bfloat16:
        return torch.matmul(x.float(), y.float()).to(out_dtype)
    r = torch.matmul(x, y)
    return r if out_dtype is None or r.dtype == out_dtype else r.to(out_dtype)


# Fast-weight gradients summed in f32 by the GEMM epilogue (False: every contribution is a bf16 tensor that autograd adds up).
CAST_ACC = os.environ.get("DTTT_CAST_ACC", "1") == "1"
ACC_MISSES = None       # a dict while a profile wants to know which products could not use the buffer (tools/step_profile.py)
ACC_DIRECT = [0]        # ordinary gradients that reached a tracked copy's backward node


class _CastAcc(torch.autograd.Function):
    """The bf16 compute copy of an f32 per-sequence weight.  The copy carries ``grad_acc``, a one-slot holder: in a backward
    that is not being recorded every product that owes the copy a gradient adds it into one f32 buffer through the GEMM's
    accumulating epilogue (``_MM.backward``) and hands autograd nothing; this node's backward, which runs once all of them
    have reported, returns the buffer.  It replaces one bf16 tensor per contribution, the additions between them and the
    cast back to f32 (the meta-gradient reaches a chunk's fast weights through the read, the clean stream and the write:
    reference src/ttt/chunk_scan.py:604-625)."""

    @staticmethod
    def forward(ctx, w, holder, lo):
        ctx.set_materialize_grads(False)
        ctx.holder = holder
        return w.to(torch.bfloat16) if lo is None else lo.view_as(lo)

    @staticmethod
    def backward(ctx, g):
        acc, ctx.holder[0] = ctx.holder[0], None
        if acc is not None and ctx.holder[1] != _graph_task():
            acc = None                                  # left behind by an earlier backward that never reached this node
        if acc is None:
            return (None if g is None else g.to(torch.float32)), None, None
        if g is not None:
            ACC_DIRECT[0] += 1
            acc = acc + g if torch.is_grad_enabled() else acc.add_(g)
        return acc, None, None


_graph_task = getattr(torch._C, "_current_graph_task_id", lambda: -1)     # which backward pass is running (-1: none)


def cast_acc(w: torch.Tensor, lo: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``w.to(bfloat16)`` for an f32 ``[B, in, out]`` weight that wants its gradient summed in f32 (see ``_CastAcc``);
    ``lo``: that copy if the kernel that produced ``w`` already wrote it."""
    holder = [None, -1]                                  # the buffer, and the backward pass that is filling it
    c = _CastAcc.apply(w, holder, None if lo is None else lo.detach())
    c.grad_acc = holder
    return c


def _acc_into(holder, shape, a, b, ta, tb) -> bool:
    """Add ``op(a) @ op(b)`` to the f32 buffer of ``holder`` (created by the first product); False if this backward has to
    return an ordinary gradient instead (it is being recorded, or it is the inner step's own gradient)."""
    from .functional import _INNER_BACKWARD
    if holder is None or torch.is_grad_enabled() or _INNER_BACKWARD[0]:
        return False
    M = a.shape[-1] if ta else a.shape[-2]
    N = b.shape[-2] if tb else b.shape[-1]
    if not (_kernel_ok(a) and _kernel_ok(b)) or a.dim() != len(shape) or b.dim() != len(shape) or (a.shape[0], M, N) != tuple(shape):
        if ACC_MISSES is not None:
            key = (tuple(a.shape), str(a.dtype), tuple(b.shape), str(b.dtype), ta, tb, tuple(shape))
            ACC_MISSES[key] = ACC_MISSES.get(key, 0) + 1
        return False
    task = _graph_task()
    if holder[0] is None or holder[1] != task:
        # the first product of this backward pass (a buffer of another pass, one that took a gradient w.r.t. something
        # downstream of the weights and so never ran the copy's own node, is dropped)
        holder[0], holder[1] = gemm_raw(a, b, ta, tb, torch.float32), task
    else:
        gemm_raw(a, b, ta, tb, torch.float32, out=holder[0], accumulate=True)
    return True


class _MM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, a, b, ta, tb, out_dtype):
        ctx.save_for_backward(a, b)
        ctx.ta, ctx.tb = ta, tb
        ctx.acc_a, ctx.acc_b = getattr(a, "grad_acc", None), getattr(b, "grad_acc", None)
        return gemm_raw(a, b, ta, tb, out_dtype)

    @staticmethod
    def backward(ctx, g):
        a, b = ctx.saved_tensors
        ta, tb = ctx.ta, ctx.tb
        g = g if g.dtype == torch.bfloat16 else g.to(torch.bfloat16)
        ga = gb = None
        # y = op(a) op(b);  d op(a) = g op(b)^T,  d op(b) = op(a)^T g
        if ctx.needs_input_grad[0]:
            args = (b, g, tb, True) if ta else (g, b, False, not tb)
            if not _acc_into(ctx.acc_a, a.shape, *args):
                ga = mm(*args)
                if ga.dim() > a.dim():
                    ga = ga.sum(0)
        if ctx.needs_input_grad[1]:
            args = (g, a, True, ta) if tb else (a, g, not ta, False)
            if not _acc_into(ctx.acc_b, b.shape, *args):
                gb = mm(*args)
                if gb.dim() > b.dim():
                    gb = gb.sum(0)
        return ga, gb, None, None, None


def mm(a: torch.Tensor, b: torch.Tensor, ta: bool = False, tb: bool = False,
       out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """``op(a) @ op(b)``, differentiable (to any order); see the module docstring."""
    if _kernel_ok(a) and _kernel_ok(b) and a.dim() >= 2 and b.dim() >= 2 and a.dim() <= 3 and b.dim() <= 3:
        od = out_dtype or torch.bfloat16
        if torch.is_grad_enabled() and (a.requires_grad or b.requires_grad):
            return _MM.apply(a, b, ta, tb, od)
        return gemm_raw(a, b, ta, tb, od)
    return _torch_mm(a, b, ta, tb, out_dtype)


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w (+ bias)`` with ``w [in, out]``; ``x`` of any leading shape."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if w.dtype != x2.dtype:
        w = w.to(x2.dtype)
    y = mm(x2, w)
    if bias is not None:
        y = y + bias.to(y.dtype)
    return y.view(*lead, w.shape[-1])
