"""Worker of the tensor-parallel fused-kernel test: all-gather -> GEMM and GEMM -> reduce-scatter over peer memory on N
GPUs against plain matmuls of the unsharded operands, forward and backward, several calls in a row (buffers alternate)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from dttt_b200.ops import _lib  # noqa: E402
from dttt_b200.parallel import tp  # noqa: E402
from dttt_b200.parallel.mesh import init_distributed  # noqa: E402


def rel(a, b):
    return (a.float() - b.float()).abs().max().item() / (b.float().abs().max().item() + 1e-12)


def main():
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    rank, world, local = init_distributed("nccl", timeout_s=120)
    dev = torch.device("cuda", local)
    ws = tp.Workspace(dist.group.WORLD, dev, nbytes=256 << 20)
    gen = torch.Generator(device="cpu")
    worst = 0.0
    for it, (M, K, N) in enumerate([(1024, 512, 768), (1024, 512, 768), (1024, 512, 768), (2048, 1024, 512), (1024, 512, 768)]):
        gen.manual_seed(100 + it)
        X = (torch.randn(M, K, generator=gen)).to(dev, torch.bfloat16)
        W = (torch.randn(K, N, generator=gen) * 0.05).to(dev, torch.bfloat16)
        G = torch.randn(M, N, generator=gen).to(dev, torch.bfloat16)
        rows, nc, kc = M // world, N // world, K // world
        # column parallel: rows of X sharded, columns of W sharded
        xs = X[rank * rows:(rank + 1) * rows].clone().requires_grad_(True)
        wc = W[:, rank * nc:(rank + 1) * nc].contiguous().requires_grad_(True)
        y = tp.column_linear(xs, wc, ws)
        gx, gw = torch.autograd.grad(y, (xs, wc), G[:, rank * nc:(rank + 1) * nc].contiguous())
        X32, W32 = X.float().requires_grad_(), W.float().requires_grad_()
        Y32 = X32 @ W32
        gX32, gW32 = torch.autograd.grad(Y32, (X32, W32), G.float())
        errs = [rel(y, Y32[:, rank * nc:(rank + 1) * nc]), rel(gx, gX32[rank * rows:(rank + 1) * rows]), rel(gw, gW32[:, rank * nc:(rank + 1) * nc])]
        # row parallel: columns of X (the contraction) sharded, rows of W sharded, output rows scattered
        xr = X[:, rank * kc:(rank + 1) * kc].contiguous().requires_grad_(True)
        wr = W[rank * kc:(rank + 1) * kc].contiguous().requires_grad_(True)
        res = G[rank * rows:(rank + 1) * rows].contiguous()
        y2 = tp.row_linear(xr, wr, ws, residual=res)
        gx2, gw2 = torch.autograd.grad(y2, (xr, wr), G[rank * rows:(rank + 1) * rows].contiguous())
        errs += [rel(y2, (Y32 + G.float())[rank * rows:(rank + 1) * rows]), rel(gx2, gX32[:, rank * kc:(rank + 1) * kc]),
                 rel(gw2, gW32[rank * kc:(rank + 1) * kc])]
        torch.cuda.synchronize()
        _lib.check_status()
        worst = max(worst, max(errs))
        if max(errs) > 3e-2:
            print(f"rank {rank} call {it} errors {errs}", flush=True)
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        print(f"TP_WORST_REL_ERR {t.item():.5f}", flush=True)
    dist.barrier()
    dist.destroy_process_group()
    sys.exit(0 if t.item() < 3e-2 else 1)


if __name__ == "__main__":
    main()
