"""Time the fused compute+collective kernels on N GPUs of one node against their rooflines and against the
unfused baseline (NCCL collective, then the plain GEMM / optimiser kernel).

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port 29533 \
        -m dttt_b200.tools.comm_bench [--rows 49152] [--out comm_bench.jsonl]

One JSON line per case (rank 0 prints).  Timing: CUDA events on the launching stream of every rank, three warm-up
calls, the median of ``--iters`` calls with a barrier before each, then the MAX over ranks.  Roofline of a fused
kernel = the slower of (FLOPs / measured cuBLAS bf16 burst) and (bytes that must cross NVLink per GPU / 770 GB/s,
the measured one-direction peer copy rate on this pool); for the optimiser kernels, bytes over NVLink versus local
HBM bytes over the measured copy bandwidth.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
NVLINK = 770e9


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


def timed(fn, iters, group):
    for _ in range(3):
        fn()
    ts = []
    for _ in range(iters):
        dist.barrier(group=group)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    t = torch.tensor([ts[len(ts) // 2]], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t.item()


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.comm_bench")
    ap.add_argument("--rows", type=int, default=49152)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    ap.add_argument("--only", default="", help="run one family: tp (gemm_ag / gemm_rs), wg (weight-gather GEMM), optim")
    a = ap.parse_args(argv)
    sys.path.insert(0, ROOT)
    from dttt_b200.ops import _lib, gemm
    from dttt_b200.parallel import symm, tp
    from dttt_b200.parallel.mesh import init_distributed

    rank, world, local = init_distributed("nccl", timeout_s=300)
    dev = torch.device("cuda", local)
    group = dist.group.WORLD
    hbm, flops, src = peaks()
    lines = []

    def out(d):
        d.update(n_gpus=world, peaks=src)
        if rank == 0:
            lines.append(json.dumps(d))
            print(lines[-1], flush=True)

    M = a.rows - a.rows % (128 * world)
    rows = M // world
    want = lambda fam: a.only in ("", fam)
    # ---- FSDP weight all-gather -> GEMM: the weight lies in a flat space cut evenly over the ranks
    if want("wg"):
        import ctypes
        from dttt_b200.parallel.wgather import WeightGather
        for name, K, N in (("qkv", 2048, 3072), ("mlp_up", 2048, 8192), ("mlp_down", 8192, 2048)):
            n_w = K * N
            shard_w = n_w // world
            pbw = symm.PeerBuffer(n_w * 2, group, dev)
            pbw.tensor(0, n_w, torch.bfloat16).normal_(0, 0.02)
            table = (ctypes.c_void_p * world)(*[ctypes.c_void_p(p_ + r_ * shard_w * 2) for r_, p_ in enumerate(pbw.ptrs)])
            wgr = WeightGather(table, shard_w, world, rank, dev, n_w, max(K, N))
            x = torch.randn(M, K, device=dev, dtype=torch.bfloat16)
            mine = pbw.tensor(rank * shard_w * 2, shard_w, torch.bfloat16)
            full = torch.empty(n_w, device=dev, dtype=torch.bfloat16)
            torch.cuda.synchronize(); dist.barrier(group=group)
            t_f = timed(lambda: wgr.gemm(x, (K, N), 0, False), a.iters, group)

            def base_wg():
                dist.all_gather_into_tensor(full, mine, group=group)
                gemm.gemm_raw(x, full.view(K, N), False, False)
            t_b = timed(base_wg, a.iters, group)
            t_g = timed(lambda: gemm.gemm_raw(x, full.view(K, N), False, False), a.iters, group)
            fl = 2.0 * M * K * N
            link = (n_w - shard_w) * 2.0
            roof = max(fl / flops, link / NVLINK) * 1e3
            out({"kernel": "gemm_wg (weight all-gather -> GEMM)", "case": name, "M": M, "K": K, "N": N, "ms": t_f, "ms_nccl_then_gemm": t_b,
                 "ms_gemm_alone": t_g, "speedup_vs_unfused": t_b / t_f, "roofline_ms": roof, "frac_of_roofline": roof / t_f,
                 "tflops": fl / t_f / 1e9, "nvlink_gbs_in": link / t_f / 1e6})
            torch.cuda.synchronize(); dist.barrier(group=group)
            del wgr, pbw
    if not (want("tp") or want("optim")):
        torch.cuda.synchronize()
        _lib.check_status()
        if a.out and rank == 0:
            with open(a.out, "w") as fh:
                fh.write("\n".join(lines) + "\n")
        dist.barrier(group=group)
        dist.destroy_process_group()
        return 0
    ws = tp.Workspace(group, dev, nbytes=6 << 30)
    # ---- all-gather -> GEMM (column parallel): QKV and MLP up of the 1B model
    for name, K, N in ((("qkv", 2048, 3072), ("mlp_up", 2048, 8192)) if want("tp") else ()):
        Nl = N // world
        xs = torch.randn(rows, K, device=dev, dtype=torch.bfloat16)
        w = (torch.randn(K, Nl, device=dev) * 0.02).to(torch.bfloat16)
        full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)
        t_f = timed(lambda: tp.ag_gemm(ws, xs, w), a.iters, group)

        def base():
            dist.all_gather_into_tensor(full, xs, group=group)
            gemm.gemm_raw(full, w, False, False)
        t_b = timed(base, a.iters, group)
        fl = 2.0 * M * K * Nl
        link = (M - rows) * K * 2.0
        roof = max(fl / flops, link / NVLINK) * 1e3
        out({"kernel": "gemm_ag (all-gather -> GEMM)", "case": name, "M": M, "K": K, "N_local": Nl, "ms": t_f, "ms_nccl_then_gemm": t_b,
             "speedup_vs_unfused": t_b / t_f, "roofline_ms": roof, "frac_of_roofline": roof / t_f, "tflops": fl / t_f / 1e9,
             "nvlink_gbs_in": link / t_f / 1e6})
    # ---- GEMM -> reduce-scatter (row parallel): attention out and MLP down
    for name, K, N in ((("attn_out", 2048, 2048), ("mlp_down", 8192, 2048)) if want("tp") else ()):
        Kl = K // world
        x = torch.randn(M, Kl, device=dev, dtype=torch.bfloat16)
        w = (torch.randn(Kl, N, device=dev) * 0.02).to(torch.bfloat16)
        part = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        mine = torch.empty(rows, N, device=dev, dtype=torch.bfloat16)
        t_f = timed(lambda: tp.gemm_rs(ws, x, w), a.iters, group)

        def base():
            gemm.gemm_raw(x, w, False, False, out=part)
            dist.reduce_scatter_tensor(mine, part, group=group)
        t_b = timed(base, a.iters, group)
        fl = 2.0 * M * Kl * N
        link = (M - rows) * N * 2.0
        roof = max(fl / flops, link / NVLINK) * 1e3
        out({"kernel": "gemm_rs (GEMM -> reduce-scatter) + slot_reduce", "case": name, "M": M, "K_local": Kl, "N": N, "ms": t_f,
             "ms_gemm_then_nccl": t_b, "speedup_vs_unfused": t_b / t_f, "roofline_ms": roof, "frac_of_roofline": roof / t_f,
             "tflops": fl / t_f / 1e9, "nvlink_gbs_out": link / t_f / 1e6})
    if not want("optim"):
        torch.cuda.synchronize()
        _lib.check_status()
        if a.out and rank == 0:
            with open(a.out, "w") as fh:
                fh.write("\n".join(lines) + "\n")
        dist.barrier(group=group)
        dist.destroy_process_group()
        return 0
    # ---- optimiser step collectives: reduce-scatter + sum of squares, AdamW + all-gather (1.4 B parameters)
    n = 1437157376 // (64 * world) * (64 * world)
    shard = n // world
    pb = symm.PeerBuffer(n * 4 + n * 2, group, dev)
    grad = pb.tensor(0, n, torch.float32)
    grad.normal_()
    gtab, ltab = pb.ptr_table(0), pb.ptr_table(n * 4)
    gs = torch.empty(shard, device=dev)
    sumsq = torch.zeros(1, device=dev)
    torch.cuda.synchronize(); dist.barrier(group=group)
    t_f = timed(lambda: symm.reduce_scatter_sumsq(gtab, world, rank, rank * shard, shard, 1.0, gs, sumsq), a.iters, group)

    def base_rs():
        dist.reduce_scatter_tensor(gs, grad, group=group)
        sumsq.copy_(gs.pow(2).sum())
    t_b = timed(base_rs, a.iters, group)
    link = (world - 1) * shard * 4.0
    roof = max(link / NVLINK, (shard * 4.0 * 2) / hbm) * 1e3
    out({"kernel": "reduce_scatter_sumsq", "elements": n, "ms": t_f, "ms_nccl_then_norm": t_b, "speedup_vs_unfused": t_b / t_f,
         "roofline_ms": roof, "frac_of_roofline": roof / t_f, "nvlink_gbs_in": link / t_f / 1e6})
    p_, m_, v_ = (torch.randn(shard, device=dev) for _ in range(3))
    v_.abs_()
    lo = pb.tensor(n * 4, n, torch.bfloat16)
    t_f = timed(lambda: symm.adamw_allgather(p_, m_, v_, gs, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0, ltab, world, rank, rank * shard, True),
                a.iters, group)
    from dttt_b200.ops import kernels

    def base_adam():
        kernels.adamw(p_, m_, v_, gs, 1e-4, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0)
        dist.all_gather_into_tensor(lo, p_.to(torch.bfloat16), group=group)
    t_b = timed(base_adam, a.iters, group)
    link = (world - 1) * shard * 2.0
    roof = max(link / NVLINK, (shard * 4.0 * 7) / hbm) * 1e3
    out({"kernel": "adamw_allgather", "elements": n, "ms": t_f, "ms_adamw_then_nccl": t_b, "speedup_vs_unfused": t_b / t_f,
         "roofline_ms": roof, "frac_of_roofline": roof / t_f, "nvlink_gbs_out": link / t_f / 1e6})
    torch.cuda.synchronize()
    _lib.check_status()
    if a.out and rank == 0:
        with open(a.out, "w") as fh:
            fh.write("\n".join(lines) + "\n")
    dist.barrier(group=group)
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
