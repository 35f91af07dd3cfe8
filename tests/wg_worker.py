"""Worker of the weight-gather GEMM test: every rank holds one slice of a flat bf16 parameter space in peer memory; products
with weights that lie anywhere in that space (inside one slice, across a slice boundary, across several) are compared with
torch on the full weight."""
import ctypes
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from dttt_b200.ops import _lib  # noqa: E402
from dttt_b200.parallel.mesh import init_distributed  # noqa: E402
from dttt_b200.parallel.symm import PeerBuffer  # noqa: E402
from dttt_b200.parallel.wgather import WeightGather  # noqa: E402


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = init_distributed("nccl", timeout_s=120)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    # weights [rows, cols] laid back to back (64-element aligned starts) in a flat space cut into `world` equal slices
    shapes = [(256, 512), (1024, 384), (128, 2048), (2048, 2048), (192, 72), (2048, 8192)]
    offs, n = [], 0
    for r_, c_ in shapes:
        offs.append(n)
        n += -(-(r_ * c_) // 64) * 64
    pad = 64 * world
    total = -(-n // pad) * pad
    shard = total // world
    full = (0.5 * torch.randn(total, generator=torch.Generator().manual_seed(7))).to(torch.bfloat16).to(dev)
    peer = PeerBuffer(total * 2, None, dev)
    mine = peer.tensor(0, total, torch.bfloat16)
    mine.fill_(float("nan"))                                   # nothing outside the own slice may be used
    mine[rank * shard:(rank + 1) * shard].copy_(full[rank * shard:(rank + 1) * shard])
    table = (ctypes.c_void_p * world)(*[ctypes.c_void_p(p + r * shard * 2) for r, p in enumerate(peer.ptrs)])
    wg = WeightGather(table, shard, world, rank, dev, max(a * b for a, b in shapes), max(max(s) for s in shapes))
    torch.cuda.synchronize()
    dist.barrier()
    worst = 0.0
    g = torch.Generator(device="cuda").manual_seed(11 + rank)
    for (rows, cols), off in zip(shapes, offs):
        W = full[off:off + rows * cols].view(rows, cols).float()
        for M in (512, 1000, 4096):
            x = torch.randn(M, rows, device=dev, generator=g).to(torch.bfloat16)
            y = wg.gemm(x, (rows, cols), off, False)
            want = x.float() @ W
            worst = max(worst, ((y.float() - want).abs().max() / want.abs().max()).item())
            gy = torch.randn(M, cols, device=dev, generator=g).to(torch.bfloat16)
            gx = wg.gemm(gy, (rows, cols), off, True)
            want = gy.float() @ W.t()
            worst = max(worst, ((gx.float() - want).abs().max() / want.abs().max()).item())
        # f32 accumulation into an existing buffer (the form a gradient product would use)
        x = torch.randn(256, rows, device=dev, generator=g).to(torch.bfloat16)
        acc = torch.ones(256, cols, dtype=torch.float32, device=dev)
        wg.gemm(x, (rows, cols), off, False, out=acc, accumulate=True)
        want = 1.0 + x.float() @ W
        worst = max(worst, ((acc - want).abs().max() / want.abs().max()).item())
    torch.cuda.synchronize()
    _lib.check_status()
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    dist.barrier()
    if rank == 0:
        print(f"WG_WORST_REL_ERR {t.item():.3e}", flush=True)
    assert t.item() < 2e-2, t.item()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
