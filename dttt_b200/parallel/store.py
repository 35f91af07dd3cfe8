"""Sharded parameter storage: f32 masters and optimiser moments split over the FSDP group, full
compute copies and full f32 gradient buffers on every rank.

The reference keeps f32 masters and Adam moments sharded on the last divisible axis of every array
and lets XLA all-gather bf16 copies per use (``src/ttt/sharding.py:39-52``, ``train.py:678-707``).  On a
180 GB part the full bf16 copy of a 1.4 B model is 3 GB, so this store gathers every compute copy once
per step and keeps it resident; what is sharded is what is large and persistent: the f32 master, the
two Adam moments (``1/fsdp`` of ``12 bytes x params`` per rank).

Layout: parameters are laid out back to back in two flat index spaces, *big* (matrices: compute dtype
copies) and *small* (norm weights, biases, gates, scalars: used in f32).  Every parameter is a shaped
view into the flat buffers.  Rank ``r`` of the FSDP group owns the flat slice
``[r * n / fsdp, (r + 1) * n / fsdp)`` of each space, regardless of parameter boundaries.

A step is: ``zero_grad`` -> forward/backward (gradients land in ``grad_*`` by GEMM-epilogue
accumulation or ``fold_grads``) -> ``reduce_grads`` (reduce-scatter over fsdp, all-reduce over dp) ->
optimiser on the shards (``optim.ShardedAdamW``) -> ``sync_compute`` (cast + all-gather).
"""
from __future__ import annotations

import math
from collections import OrderedDict
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..models.params import is_small
from .mesh import Mesh

ALIGN = 64          # elements; keeps every parameter view 128-byte aligned in bf16


class ParamStore:
    def __init__(self, spec: "OrderedDict[str, Tuple[Tuple[int, ...], str]]", mesh: Mesh, compute_dtype: torch.dtype,
                 device: torch.device, trainable: bool = True, fused_comm: bool = True, tp_ctx=None):
        """``spec`` holds the shapes THIS rank stores (tensor-parallel slices when ``mesh.tp > 1``, see
        ``models.params.tp_layout``); ``tp_ctx``: the ``parallel.tp.TPContext`` the sliced weights are used through."""
        self.spec, self.mesh, self.dtype, self.device = spec, mesh, compute_dtype, device
        self.trainable = trainable
        self.tp_ctx = tp_ctx
        from ..models.params import tp_layout
        self.tp_layout = {n: tp_layout(n) for n in spec} if mesh.tp > 1 else {}
        self.fs = mesh.fsdp
        self.slots: Dict[str, Tuple[str, int, int, Tuple[int, ...]]] = {}      # name -> (space, offset, numel, shape)
        offs = {"big": 0, "small": 0}
        for name, (shape, _) in spec.items():
            space = "small" if is_small(name) else "big"
            n = math.prod(shape) if shape else 1
            self.slots[name] = (space, offs[space], n, tuple(shape))
            offs[space] += -(-n // ALIGN) * ALIGN
        pad = ALIGN * self.fs
        self.n = {k: max(pad, -(-v // pad) * pad) for k, v in offs.items()}
        self.shard_n = {k: v // self.fs for k, v in self.n.items()}
        f32 = torch.float32
        # With more than one FSDP rank on GPUs the compute copies and the gradient buffers live in peer-accessible
        # memory (parallel.symm): the fused reduce-scatter / optimiser / all-gather kernels read and write the other
        # ranks' copies directly over NVLink.  Otherwise they are ordinary tensors and the collectives are NCCL / gloo.
        self.peer = None
        # (under tensor parallelism the FSDP group of a rank is the ranks that hold the same slices; the gradients of whole
        # parameters are first summed over the TP group by NCCL, then every group runs the same fused kernels)
        self.fused = bool(fused_comm and trainable and self.fs > 1 and device.type == "cuda")
        if self.fused:
            from .symm import PeerBuffer
            lo_big = self.n["big"] * torch.empty(0, dtype=compute_dtype).element_size()
            self._off = {"lo_big": 0, "lo_small": lo_big}
            self._off["grad_big"] = self._off["lo_small"] + self.n["small"] * 4
            self._off["grad_small"] = self._off["grad_big"] + self.n["big"] * 4
            total = self._off["grad_small"] + self.n["small"] * 4
            self.peer = PeerBuffer(total, mesh.fsdp_group, device)
            self.lo = {"big": self.peer.tensor(self._off["lo_big"], self.n["big"], compute_dtype),
                       "small": self.peer.tensor(self._off["lo_small"], self.n["small"], f32)}
            self.grad = {k: self.peer.tensor(self._off["grad_" + k], self.n[k], f32) for k in ("big", "small")}
            self._grad_tables = {k: self.peer.ptr_table(self._off["grad_" + k]) for k in ("big", "small")}
            self._lo_tables = {k: self.peer.ptr_table(self._off["lo_" + k]) for k in ("big", "small")}
            self.sumsq = torch.zeros(2, dtype=f32, device=device)
            self._bar = torch.zeros(1, dtype=f32, device=device)
        else:
            self.lo = {"big": torch.zeros(self.n["big"], dtype=compute_dtype, device=device),
                       "small": torch.zeros(self.n["small"], dtype=f32, device=device)}
            self.grad = {k: torch.zeros(self.n[k], dtype=f32, device=device) for k in ("big", "small")} if trainable else None
        self.sharded_names: set = set()        # matrices whose compute copy is gathered per use (enable_shard_compute)
        self.wgather = None
        ns = self.shard_n["big"] + self.shard_n["small"]
        self.master = torch.zeros(ns, dtype=f32, device=device)                   # [big shard | small shard]
        self.grad_shard = torch.zeros(ns, dtype=f32, device=device) if trainable else None

    # ---- per-use weight gather (parallel.wgather)
    def enable_shard_compute(self, names) -> None:
        """From now on the compute copies of ``names`` (stacked matrices ``[layers, in, out]`` of the big space) are kept
        current only inside each rank's own flat slice: the optimiser stops pushing them to the peers and every product
        with one of them gathers it inside the GEMM (``parallel.wgather``).  Needs the peer-memory layout (``fused``)."""
        if not self.fused or self.mesh.tp > 1 or self.dtype != torch.bfloat16:
            raise ValueError("shard_compute needs fused_comm on a GPU FSDP group of more than one rank, bf16, no tensor parallelism")
        import ctypes
        from .wgather import WeightGather
        names = [n for n in names if n in self.slots and self.slots[n][0] == "big" and len(self.slots[n][3]) == 3]
        if not names:
            return
        es = 2
        base = self._off["lo_big"]
        table = (ctypes.c_void_p * self.fs)(*[ctypes.c_void_p(p + base + r * self.shard_n["big"] * es) for r, p in enumerate(self.peer.ptrs)])
        biggest = max(self.slots[n][3][1] * self.slots[n][3][2] for n in names)
        rows = max(max(self.slots[n][3][1], self.slots[n][3][2]) for n in names)
        self.wgather = WeightGather(table, self.shard_n["big"], self.fs, self.mesh.fsdp_index, self.device, biggest, rows)
        self.sharded_names = {n for n in names if self.wgather.supports(self.slots[n][3][1:])
                              and self.wgather.supports(self.slots[n][3][1:][::-1])}
        self._lo_self_tables = {k: (ctypes.c_void_p * 1)(ctypes.c_void_p(self.peer.local + self._off["lo_" + k])) for k in ("big", "small")}

    def forget_foreign_compute(self) -> None:
        """Overwrite, in this rank's compute buffer, what other ranks own of the per-use gathered matrices (NaN), so that
        anything that read them without gathering would show.  A test aid; the training path never reads those ranges."""
        lo, hi = self.shard_range("big")
        for n in self.sharded_names:
            _, off, cnt, _ = self.slots[n]
            for a, b in ((off, min(off + cnt, lo)), (max(off, hi), off + cnt)):
                if a < b:
                    self.lo["big"][a:b].fill_(float("nan"))

    # ---- geometry
    def tp_replicated_ranges(self) -> Dict[str, List[Tuple[int, int]]]:
        """Per space, the merged ``[start, end)`` ranges of the flat buffers that hold parameters every rank of a
        tensor-parallel group keeps whole: their gradients are partial sums over the group's sequences."""
        out: Dict[str, List[Tuple[int, int]]] = {"big": [], "small": []}
        for name, (space, off, n, _) in self.slots.items():
            if self.tp_layout.get(name) is None:
                end = -(-(off + n) // ALIGN) * ALIGN
                if out[space] and out[space][-1][1] == off:
                    out[space][-1] = (out[space][-1][0], end)
                else:
                    out[space].append((off, end))
        return out

    def shard_range(self, space: str) -> Tuple[int, int]:
        r = self.mesh.fsdp_index
        return r * self.shard_n[space], (r + 1) * self.shard_n[space]

    def master_part(self, space: str, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        buf = self.master if buf is None else buf
        nb = self.shard_n["big"]
        return buf[:nb] if space == "big" else buf[nb:]

    def segments(self) -> List[Tuple[str, int, int]]:
        """``(name, start, end)`` ranges of this rank's master shard (indices into ``self.master``).  Ends are rounded
        up to the slot alignment (the padding holds zeros and stays zero under AdamW), so every range is a whole
        number of 16-byte vectors."""
        out = []
        for name, (space, off, n, _) in self.slots.items():
            lo, hi = self.shard_range(space)
            a, b = max(off, lo), min(-(-(off + n) // ALIGN) * ALIGN, hi)
            if a < b:
                base = 0 if space == "big" else self.shard_n["big"]
                out.append((name, base + a - lo, base + b - lo))
        return out

    def space_of_master_index(self, idx: int) -> Tuple[str, int]:
        """``(space, flat offset in that space)`` of an index into this rank's master shard."""
        nb = self.shard_n["big"]
        if idx < nb:
            return "big", self.shard_range("big")[0] + idx
        return "small", self.shard_range("small")[0] + idx - nb

    def barrier(self) -> None:
        """Stream-ordered barrier over the FSDP group (a one-element all-reduce)."""
        if self.fs > 1:
            dist.all_reduce(self._bar, group=self.mesh.fsdp_group)

    # ---- views
    def lo_view(self, name: str) -> torch.Tensor:
        space, off, n, shape = self.slots[name]
        return self.lo[space][off:off + n].view(shape)

    def grad_view(self, name: str) -> torch.Tensor:
        space, off, n, shape = self.slots[name]
        return self.grad[space][off:off + n].view(shape)

    def names(self):
        return self.slots.keys()

    # ---- filling
    def load_full(self, name: str, value: torch.Tensor) -> None:
        """Set parameter ``name`` from a full f32 tensor (every rank passes the same values)."""
        space, off, n, shape = self.slots[name]
        lay = self.tp_layout.get(name)
        if lay is not None and tuple(value.shape) != tuple(shape):
            from ..models.params import tp_slice
            value = tp_slice(name, value, self.mesh.tp, self.mesh.tp_index)      # a full tensor (checkpoint): keep this rank's slice
        v = value.to(device=self.device, dtype=torch.float32).reshape(-1)
        assert v.numel() == n, (name, tuple(value.shape), shape)
        self.lo[space][off:off + n].copy_(v)
        lo, hi = self.shard_range(space)
        a, b = max(off, lo), min(off + n, hi)
        if a < b:
            self.master_part(space)[a - lo:b - lo].copy_(v[a - off:b - off])

    def gather_full(self, name: str, buf: Optional[torch.Tensor] = None) -> torch.Tensor:
        """The full f32 value of ``name`` assembled from the master shards (collective over the FSDP group).
        ``buf``: another sharded buffer laid out like the master (an Adam moment)."""
        space, off, n, shape = self.slots[name]
        part = self.master_part(space, buf)
        if self.fs == 1:
            local = part[off:off + n].view(shape).clone()
        else:
            full = torch.empty(self.n[space], dtype=torch.float32, device=self.device)
            dist.all_gather_into_tensor(full, part.contiguous(), group=self.mesh.fsdp_group)
            local = full[off:off + n].view(shape).clone()
        lay = self.tp_layout.get(name)
        if lay is None:
            return local
        parts = [torch.empty_like(local) for _ in range(self.mesh.tp)]           # the whole tensor from the group's slices
        dist.all_gather(parts, local, group=self.mesh.tp_group)
        return torch.cat(parts, dim=lay[1])

    # ---- the step's collectives
    def zero_grad(self) -> None:
        for g in self.grad.values():
            g.zero_()

    def reduce_grads(self) -> None:
        """Sum the full gradient buffers over every data rank and leave this rank's slice in ``grad_shard``."""
        m = self.mesh
        if m.tp > 1:
            for space, ranges in self.tp_replicated_ranges().items():
                for a, b in ranges:
                    dist.all_reduce(self.grad[space][a:b], op=dist.ReduceOp.SUM, group=m.tp_group)
        if self.fused:
            # one kernel per space: every rank pulls its slice of every peer's gradient buffer over NVLink, sums,
            # and accumulates the slice's squared norm; no library collective.
            from . import symm
            self.barrier()                                   # every rank's backward has finished writing its buffer
            self.sumsq.zero_()
            for i, space in enumerate(("big", "small")):
                lo, hi = self.shard_range(space)
                symm.reduce_scatter_sumsq(self._grad_tables[space], self.fs, m.fsdp_index, lo, hi - lo, 1.0,
                                          self.master_part(space, self.grad_shard), self.sumsq[i:i + 1])
                if m.dp > 1:
                    dist.all_reduce(self.master_part(space, self.grad_shard), op=dist.ReduceOp.SUM, group=m.dp_group)
            return
        for space in ("big", "small"):
            out = self.master_part(space, self.grad_shard)
            g = self.grad[space]
            if self.fs > 1:
                dist.reduce_scatter_tensor(out, g, op=dist.ReduceOp.SUM, group=m.fsdp_group)
            else:
                out.copy_(g)
            if m.dp > 1:
                dist.all_reduce(out, op=dist.ReduceOp.SUM, group=m.dp_group)

    def sync_compute(self) -> None:
        """Refresh the compute copies from the (updated) master shards: cast, then all-gather."""
        m = self.mesh
        for space in ("big", "small"):
            lo, hi = self.shard_range(space)
            src = self.master_part(space)
            self.lo[space][lo:hi].copy_(src)
            if self.fs > 1:
                dist.all_gather_into_tensor(self.lo[space], self.lo[space][lo:hi].clone(), group=m.fsdp_group)

    def all_reduce_scalar(self, x: torch.Tensor, groups=("fsdp", "dp", "tp")) -> torch.Tensor:
        m = self.mesh
        if "tp" in groups and m.tp > 1:
            dist.all_reduce(x, group=m.tp_group)
        if "fsdp" in groups and m.fsdp > 1:
            dist.all_reduce(x, group=m.fsdp_group)
        if "dp" in groups and m.dp > 1:
            dist.all_reduce(x, group=m.dp_group)
        return x


class ComputeWeights:
    """The compute view the model is run with: per-layer leaf tensors over a ``ParamStore``.

    ``get(name, layer)`` returns a detached view of the store's compute copy, marked ``requires_grad``
    when training.  Matrices carry ``grad_target = (f32 gradient view, layer)`` so the GEMM epilogue can
    accumulate first-order weight gradients in place; whatever reaches a leaf through ordinary autograd is
    added to the same buffers by ``fold_grads``."""

    def __init__(self, store: ParamStore, train: bool = True):
        self.store, self.train = store, train and store.trainable
        self.dtype = store.dtype
        self._leaves: Dict[Tuple[str, int], torch.Tensor] = {}

    def has(self, name: str) -> bool:
        return name in self.store.slots

    def get(self, name: str, layer: Optional[int] = None) -> torch.Tensor:
        key = (name, -1 if layer is None else layer)
        t = self._leaves.get(key)
        if t is None:
            base = self.store.lo_view(name)
            t = (base if layer is None else base[layer]).detach()
            if self.train:
                t.requires_grad_(True)
                if not is_small(name):
                    t.grad_target = (self.store.grad_view(name), layer)
            lay = self.store.tp_layout.get(name)
            if lay is not None and not name.endswith("bias"):
                t.tp = (lay[0], self.store.tp_ctx)
            if name in self.store.sharded_names and layer is not None:
                _, off, _, shape = self.store.slots[name]
                t.wg = (self.store.wgather, off + layer * shape[1] * shape[2])
            self._leaves[key] = t
        return t

    def grad_buffer(self, name: str) -> torch.Tensor:
        return self.store.grad_view(name)

    def fold_grads(self) -> None:
        for (name, layer), t in self._leaves.items():
            if t.grad is None:
                continue
            g = self.store.grad_view(name)
            (g if layer < 0 else g[layer]).add_(t.grad)
            t.grad = None
