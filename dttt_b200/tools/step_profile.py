"""Where one training step spends its time: phase ranges (CUDA events) and a per-kernel table.

    python -m dttt_b200.tools.step_profile --config configs/b200_1b_8k --seq-len 8192 --batch 2 [--kernels] [--trace out.json]

Runs two warm-up steps, then one step with the phase ranges of ``utils.prof`` switched on (the ranges synchronise,
so the wall time of that step is an upper bound), and with ``--kernels`` one more step under ``torch.profiler`` whose
device-time table is printed by kernel name (top 45) -- the reference gets the same view from ``--profile_dir``
traces (reference src/ttt/train.py:1096-1110).  ``--trace`` also writes the Chrome trace of that step.
"""
from __future__ import annotations

import argparse
import os
import sys
import time

import torch


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.step_profile")
    ap.add_argument("--config", default="configs/b200_1b_8k")
    ap.add_argument("--seq-len", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--kernels", action="store_true")
    ap.add_argument("--trace", default="")
    ap.add_argument("--shapes", action="store_true", help="also group the framework ops by input shapes")
    ap.add_argument("--top", type=int, default=60, help="rows of the by-shape table")
    ap.add_argument("--stacks", action="store_true", help="attribute the ATen ops' device time to the package's source lines")
    ap.add_argument("--keep-prefix-layers", type=int, default=0)
    ap.add_argument("--keep-suffix-chunks", type=int, default=0)
    a = ap.parse_args(argv)
    root = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, root)
    from dttt_b200.engine import Engine
    from dttt_b200.ops import gemm, kernels
    from dttt_b200.schema import ModelConfig, TrainConfig
    from dttt_b200.utils import prof

    dev = torch.device("cuda", 0)
    mc = ModelConfig.load(a.config if os.path.isabs(a.config) else os.path.join(root, a.config))
    tc = TrainConfig(seq_len=a.seq_len, batch_size=a.batch, steps=10000, seed=0, inner_task="causal", outer_shift=True,
                     keep_prefix_layers=a.keep_prefix_layers, keep_suffix_chunks=a.keep_suffix_chunks)
    eng = Engine(mc, tc, device=dev)
    ids = torch.randint(0, min(mc.vocab_size, 128000), (a.batch, a.seq_len))
    for s in range(2):
        t0 = time.time()
        eng.train_step(ids, s)
        torch.cuda.synchronize()
        print(f"warm-up step {s}: {time.time() - t0:.3f} s", flush=True)
    prof.enable(True)
    gemm.SHAPE_LOG = {}
    gemm.ACC_MISSES = {}
    gemm.ACC_DIRECT[0] = 0
    n0 = gemm.LAUNCHES, kernels.LAUNCHES
    t0 = time.time()
    eng.train_step(ids, 2)
    torch.cuda.synchronize()
    wall = time.time() - t0
    print(f"step with ranges: {wall:.3f} s  ({a.batch * a.seq_len / wall:.0f} tokens/s)  launches: gemm {gemm.LAUNCHES - n0[0]}, "
          f"other kernels {kernels.LAUNCHES - n0[1]}")
    print(prof.format_report(prof.report()))
    prof.enable(False)
    shapes, gemm.SHAPE_LOG = gemm.SHAPE_LOG, None
    tot = sum(2.0 * M * N * K * B * n for (M, N, K, B, *_), n in shapes.items())
    print(f"GEMM launches by problem (M, N, K, batch, A^T, B^T, f32 +=): {sum(shapes.values())} launches, {tot / 1e12:.1f} TFLOP")
    for key, n in sorted(shapes.items(), key=lambda kv: -2.0 * kv[0][0] * kv[0][1] * kv[0][2] * kv[0][3] * kv[1])[:40]:
        M, N, K, B = key[:4]
        print(f"  {str(key):46s} n={n:5d}  {2.0 * M * N * K * B * n / 1e12:8.2f} TFLOP  ({100 * 2.0 * M * N * K * B * n / tot:4.1f} %)")
    print(f"fast-weight gradient buffer: {gemm.ACC_DIRECT[0]} ordinary gradients reached a tracked copy; products that could not "
          f"use the buffer: {gemm.ACC_MISSES}")
    gemm.ACC_MISSES = None
    print(f"peak device memory: {torch.cuda.max_memory_allocated() / 2 ** 30:.1f} GiB")
    if a.kernels or a.trace:
        from torch.profiler import ProfilerActivity, profile
        extra = {}
        if a.stacks:                                      # Python frames are only attached with the verbose tracer
            extra["experimental_config"] = torch._C._profiler._ExperimentalConfig(verbose=True)
        with profile(activities=[ProfilerActivity.CPU, ProfilerActivity.CUDA], record_shapes=a.shapes or a.stacks,
                     with_stack=a.stacks, **extra) as p:
            eng.train_step(ids, 3)
            torch.cuda.synchronize()
        ka = p.key_averages()
        total = sum(e.self_device_time_total for e in ka) / 1e3
        print(f"device time by kernel / op (total {total:.1f} ms):")
        for e in sorted(ka, key=lambda e: -e.self_device_time_total)[:45]:
            print(f"  {e.key[:90]:90s} n={e.count:6d}  {e.self_device_time_total / 1e3:9.1f} ms")
        print("host time by op:")
        for e in sorted(ka, key=lambda e: -e.self_cpu_time_total)[:10]:
            print(f"  {e.key[:90]:90s} n={e.count:6d}  {e.self_cpu_time_total / 1e3:9.1f} ms")
        if a.shapes:
            print("device time by op and input shapes:")
            ks = p.key_averages(group_by_input_shape=True)
            for e in sorted(ks, key=lambda e: -e.self_device_time_total)[:a.top]:
                if e.key.startswith(("aten::", "_")):
                    print(f"  {e.key[:28]:28s} n={e.count:5d} {e.self_device_time_total / 1e3:8.1f} ms  {str(e.input_shapes)[:150]}")
        if a.stacks:
            # ATen ops by the innermost frame of this package that issued them; ops run by the autograd engine have no
            # Python frame and are listed under the backward node that contains them
            agg = {}
            for e in p.events():
                if not e.name.startswith("aten::") or e.self_device_time_total <= 0:
                    continue
                where = next((f for f in (e.stack or []) if "dttt_b200" in f), None)
                if where is None:
                    par, names = e.cpu_parent, []
                    while par is not None and len(names) < 2:
                        if not par.name.startswith("aten::"):
                            names.append(par.name[:60])
                        par = par.cpu_parent
                    where = " < ".join(names) or "(engine)"
                else:
                    where = where.split("dttt_b200/")[-1][:70]
                key = (e.name, where, str(e.input_shapes)[:80])
                t = agg.setdefault(key, [0, 0.0])
                t[0] += 1
                t[1] += e.self_device_time_total
            tot = sum(v[1] for v in agg.values()) / 1e3
            print(f"ATen ops by source ({tot:.1f} ms of device time):")
            for (name, where, shp), (n, us) in sorted(agg.items(), key=lambda kv: -kv[1][1])[:a.top]:
                print(f"  {name[:22]:22s} n={n:5d} {us / 1e3:7.2f} ms  {where:72s} {shp}")
        if a.trace:
            p.export_chrome_trace(a.trace)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
