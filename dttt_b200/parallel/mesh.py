"""Process groups: one process per GPU, ``world = dp x fsdp x tp``.

The reference shards with a JAX mesh ``{dp, fsdp}`` (``src/ttt/sharding.py:21-36``): parameters are
split over ``fsdp`` and replicated over ``dp``, the batch is split over both.  Here the same layout is
three explicit ``torch.distributed`` groups over the ranks of one job; ``tp`` (tensor parallel, an
addition of this package) is the innermost axis so a TP group sits on neighbouring GPUs.

    rank = (dp_index * fsdp + fsdp_index) * tp + tp_index

``fsdp_size = 0`` means "all ranks that are not TP" (the reference's pure 1-D mesh).  With a single
process every group is trivial and no backend is initialised.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class Mesh:
    rank: int = 0
    world: int = 1
    dp: int = 1
    fsdp: int = 1
    tp: int = 1
    dp_index: int = 0
    fsdp_index: int = 0
    tp_index: int = 0
    dp_group: Optional[object] = None
    fsdp_group: Optional[object] = None
    tp_group: Optional[object] = None
    device: torch.device = torch.device("cpu")

    @property
    def batch_ranks(self) -> int:
        """Ranks that hold different data: ``dp x fsdp`` (a TP group shares its batch)."""
        return self.dp * self.fsdp

    @property
    def batch_index(self) -> int:
        return self.dp_index * self.fsdp + self.fsdp_index

    def shape(self) -> dict:
        return {"dp": self.dp, "fsdp": self.fsdp, "tp": self.tp}


def mesh_shape(world: int, fsdp_size: int = 0, tp_size: int = 1) -> tuple:
    if tp_size < 1 or world % tp_size:
        raise ValueError(f"tp_size {tp_size} must divide the {world} ranks")
    rest = world // tp_size
    fsdp = rest if fsdp_size in (0, rest) or fsdp_size > rest else fsdp_size
    if rest % fsdp:
        raise ValueError(f"fsdp_size {fsdp} must divide {rest} (= {world} ranks / tp {tp_size})")
    return rest // fsdp, fsdp, tp_size


def init_distributed(backend: Optional[str] = None, timeout_s: Optional[int] = None) -> tuple:
    """Join the job described by ``RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT`` (torchrun) if there is
    one.  Returns ``(rank, world, local_rank)``.  ``DTTT_HEARTBEAT_TIMEOUT_S`` (or ``TTT_HEARTBEAT_TIMEOUT_S``)
    bounds every collective: a rank that stops answering ends the others with an error after it, the role
    of the reference's coordination-service heartbeat (``src/ttt/train.py:820-827``)."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1 and not dist.is_initialized():
        if backend is None:
            backend = "nccl" if torch.cuda.is_available() else "gloo"
        if timeout_s is None:
            timeout_s = int(os.environ.get("DTTT_HEARTBEAT_TIMEOUT_S", os.environ.get("TTT_HEARTBEAT_TIMEOUT_S", "600")))
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend=backend, rank=rank, world_size=world,
                                timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return rank, world, local


def make_mesh(fsdp_size: int = 0, tp_size: int = 1, device: Optional[torch.device] = None) -> Mesh:
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    dp, fsdp, tp = mesh_shape(world, fsdp_size, tp_size)
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device()) if torch.cuda.is_available() else torch.device("cpu")
    m = Mesh(rank=rank, world=world, dp=dp, fsdp=fsdp, tp=tp, device=device)
    m.tp_index = rank % tp
    m.fsdp_index = (rank // tp) % fsdp
    m.dp_index = rank // (tp * fsdp)
    if world == 1:
        return m
    # every rank must create every group, in the same order
    for d in range(dp):
        for f in range(fsdp):
            ranks = [(d * fsdp + f) * tp + t for t in range(tp)]
            g = dist.new_group(ranks) if tp > 1 else None
            if rank in ranks:
                m.tp_group = g
    for d in range(dp):
        for t in range(tp):
            ranks = [(d * fsdp + f) * tp + t for f in range(fsdp)]
            g = dist.new_group(ranks) if fsdp > 1 else None
            if rank in ranks:
                m.fsdp_group = g
    for f in range(fsdp):
        for t in range(tp):
            ranks = [(d * fsdp + f) * tp + t for d in range(dp)]
            g = dist.new_group(ranks) if dp > 1 else None
            if rank in ranks:
                m.dp_group = g
    return m
