"""Time the hand-written kernels in isolation and report them against the measured peaks.

    python -m dttt_b200.tools.kernel_bench gemm --m 8192 --n 8192 --k 8192 [--ta] [--tb] [--batch B] [--f32acc]
    python -m dttt_b200.tools.kernel_bench rmsnorm|rope|swiglu|adamw --rows R --dim D
    python -m dttt_b200.tools.kernel_bench attn --seqs 8 --cq 1024 --kn 9216 --heads 32 --kv-heads 8 --head-dim 64 [--causal]
    python -m dttt_b200.tools.kernel_bench ce --rows 2048 --k 2048 --vocab 128256
    python -m dttt_b200.tools.kernel_bench gemm_pair                                 (one CTA per tile / CTA pair / cuBLAS)
    python -m dttt_b200.tools.kernel_bench segment --seqs 2 --cq 1024 --window 7 --chunks 8   (one-launch prefix attention)
    python -m dttt_b200.tools.kernel_bench gdn --seqs 4 --cq 1024 --heads 16 --head-dim 128   (blocked gated delta rule)
    python -m dttt_b200.tools.kernel_bench suite            (the shapes of the 1B model)

Timing: CUDA events on the launching stream, 3 warm-up launches, best of ``--iters``; between timed launches a
buffer larger than L2 (256 MiB) is written so no operand is L2-resident from the previous launch.  The roofline
denominators are the measured copy bandwidth and cuBLAS bf16 burst throughput in ``MEASURED_PEAKS.json`` at the
repository root (fallback 6.65 TB/s, 1.59 PFLOP/s).  One JSON line per case; ``--once`` runs each kernel a single
time after one warm-up (the form to capture under a profiler).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return d["hbm_gbs"] * 1e9, d["bf16_tflops"] * 1e12, "measured"
    return 6.65e12, 1.59e15, "fallback"


_FLUSH = None


def flush_l2():
    global _FLUSH
    if _FLUSH is None:
        _FLUSH = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    _FLUSH.fill_(1)


def timeit(fn, iters=10, once=False):
    fn()
    if once:
        torch.cuda.synchronize()
        fn()
        torch.cuda.synchronize()
        return float("nan")
    for _ in range(2):
        fn()
    best = 1e30
    for _ in range(iters):
        flush_l2()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1))
    return best


def bench_gemm(a, out):
    from dttt_b200.ops import gemm
    M, N, K, B = a.m, a.n, a.k, a.batch
    lead = (B,) if B > 1 else ()
    A = torch.randn(*lead, *((K, M) if a.ta else (M, K)), device="cuda", dtype=torch.bfloat16)
    Bm = torch.randn(*lead, *((N, K) if a.tb else (K, N)), device="cuda", dtype=torch.bfloat16)
    C = torch.zeros(*lead, M, N, device="cuda", dtype=torch.float32) if a.f32acc else None
    fn = lambda: gemm.gemm_raw(A, Bm, a.ta, a.tb, torch.float32 if a.f32acc else torch.bfloat16, out=C, accumulate=a.f32acc)
    ms = timeit(fn, a.iters, a.once)
    hbm, flops, src = peaks()
    fl = 2.0 * M * N * K * B
    res = {"kernel": "gemm_bf16_tcgen05", "M": M, "N": N, "K": K, "batch": B, "ta": a.ta, "tb": a.tb, "f32_accumulate": a.f32acc,
           "ms": ms, "tflops": fl / ms / 1e9, "frac_of_cublas_peak": fl / (ms * 1e-3) / flops, "peaks": src}
    if a.compare and not a.once:
        X = A.transpose(-1, -2) if a.ta else A
        Y = Bm.transpose(-1, -2) if a.tb else Bm
        mt = timeit(lambda: torch.matmul(X, Y), a.iters)
        res.update(ms_cublas=mt, tflops_cublas=fl / mt / 1e9, vs_cublas=mt / ms)
    out(res)


def bench_gemm_forms(a, out):
    """The model's large plain GEMM shapes under both tile forms (128 x 256 with double-buffered accumulators, 256 x 256 with two
    row halves per B tile), one line per shape."""
    from dttt_b200.ops import gemm
    _, flops, src = peaks()
    shapes = [(49152, 8192, 2048, 1, 0, 0), (49152, 2048, 8192, 1, 0, 0), (49152, 2048, 2048, 1, 0, 0), (2048, 8192, 2048, 1, 0, 0),
              (2048, 128256, 2048, 1, 0, 1), (2048, 8192, 49152, 1, 1, 0), (1024, 8192, 2048, 2, 0, 0), (8192, 8192, 8192, 1, 0, 0)]
    for M, N, K, B, ta, tb in shapes:
        lead = (B,) if B > 1 else ()
        x = torch.randn(*lead, *((K, M) if ta else (M, K)), device="cuda", dtype=torch.bfloat16)
        w = torch.randn(*lead, *((N, K) if tb else (K, N)), device="cuda", dtype=torch.bfloat16)
        res = {"kernel": "gemm tile forms", "M": M, "N": N, "K": K, "batch": B, "ta": ta, "tb": tb, "peaks": src}
        for form, name in ((0, "ms_128x256"), (1, "ms_256x256")):
            gemm.set_tile_form(form)
            ms = timeit(lambda: gemm.gemm_raw(x, w, bool(ta), bool(tb)), a.iters)
            res[name] = ms
            res[name.replace("ms_", "tflops_")] = 2.0 * M * N * K * B / ms / 1e9
        gemm.set_tile_form(-1)
        res["speedup_256"] = res["ms_128x256"] / res["ms_256x256"]
        out(res)


def bench_elementwise(a, out):
    from dttt_b200.ops import kernels
    R, D = a.rows, a.dim
    hbm, _, src = peaks()
    x = torch.randn(R, D, device="cuda", dtype=torch.bfloat16)
    if a.cmd == "rmsnorm":
        w = torch.ones(D, device="cuda")
        y, (rstd,) = kernels._rms_fwd(x, w, 1e-6)
        g = torch.randn_like(x)
        cases = [("rmsnorm_fwd", lambda: kernels._rms_fwd(x, w, 1e-6), 2 * R * D * 2),
                 ("rmsnorm_bwd", lambda: kernels._rms_bwd(g, (x, w), (rstd,), (True, True), 1e-6), 3 * R * D * 2)]
    elif a.cmd == "swiglu":
        u, g = torch.randn_like(x), torch.randn_like(x)
        cases = [("swiglu_fwd", lambda: kernels._swiglu_fwd(x, u), 3 * R * D * 2),
                 ("swiglu_bwd", lambda: kernels._swiglu_bwd(g, (x, u), (), (True, True)), 5 * R * D * 2)]
    elif a.cmd == "rope":
        heads, d = D // 64, 64
        xx = x.view(R, heads, d)
        pos = torch.arange(R, device="cuda")
        from dttt_b200.ops import functional as Fn
        inv = Fn.inv_freq(d, 5e5, None, xx.device)
        cases = [("rope", lambda: kernels._rope_run(xx, pos, inv, 1.0), 2 * R * D * 2)]
    else:
        n = R * D
        p, m, v, g = (torch.randn(n, device="cuda") for _ in range(4))
        cases = [("adamw", lambda: kernels.adamw(p, m, v, g, 1e-3, 0.9, 0.95, 1e-8, 0.1, 0.1, 0.05, 1.0), 7 * n * 4)]
    for name, fn, nbytes in cases:
        ms = timeit(fn, a.iters, a.once)
        out({"kernel": name, "rows": R, "dim": D, "ms": ms, "gbs": nbytes / ms / 1e6, "frac_of_copy_bw": nbytes / (ms * 1e-3) / hbm, "peaks": src})


def _sdpa_fast(q, k, v, scale, causal):
    """The library path the attention kernels are compared with: torch SDPA with grouped heads; ``causal`` is aligned to the end
    of the key axis (query i sees keys j <= i + Kn - Cq)."""
    import torch.nn.functional as F
    qh, kh, vh = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
    if causal and k.shape[1] != q.shape[1]:
        from torch.nn.attention.bias import causal_lower_right
        o = F.scaled_dot_product_attention(qh, kh, vh, attn_mask=causal_lower_right(q.shape[1], k.shape[1]), scale=scale, enable_gqa=True)
    else:
        o = F.scaled_dot_product_attention(qh, kh, vh, is_causal=bool(causal), scale=scale, enable_gqa=True)
    return o.transpose(1, 2)


def bench_gemm_pair(a, out):
    """The plain GEMM on one CTA per tile against the CTA-pair form (``csrc/gemm_pair_tcgen05.cu``: two SMs share each B tile)
    and cuBLAS, on the model's shapes."""
    from dttt_b200.ops import gemm
    _, flops, src = peaks()
    shapes = [(8192, 8192, 8192, 1, 0, 0), (49152, 2048, 2048, 1, 0, 0), (49152, 8192, 2048, 1, 0, 0), (49152, 2048, 8192, 1, 0, 0),
              (2048, 8192, 2048, 1, 0, 0), (2048, 2048, 8192, 1, 0, 0), (1024, 8192, 2048, 4, 0, 0), (49152, 2048, 8192, 1, 0, 1),
              (2048, 3072, 2048, 1, 0, 0), (2048, 512, 2048, 1, 0, 0)]
    was = gemm.PAIR
    for M, N, K, B, ta, tb in shapes:
        lead = (B,) if B > 1 else ()
        x = torch.randn(*lead, *((K, M) if ta else (M, K)), device="cuda", dtype=torch.bfloat16)
        w = torch.randn(*lead, *((N, K) if tb else (K, N)), device="cuda", dtype=torch.bfloat16)
        res = {"kernel": "gemm single CTA / CTA pair", "M": M, "N": N, "K": K, "batch": B, "ta": ta, "tb": tb, "peaks": src}
        fl = 2.0 * M * N * K * B
        for pair, name in ((False, "single"), (True, "pair")):
            gemm.PAIR = pair
            ms = timeit(lambda: gemm.gemm_raw(x, w, bool(ta), bool(tb)), a.iters)
            res["ms_" + name], res["tflops_" + name] = ms, fl / ms / 1e9
        X, Y = (x.transpose(-1, -2) if ta else x), (w.transpose(-1, -2) if tb else w)
        mt = timeit(lambda: torch.matmul(X, Y), a.iters)
        res.update(ms_cublas=mt, tflops_cublas=fl / mt / 1e9, pair_vs_single=res["ms_single"] / res["ms_pair"], pair_vs_cublas=mt / res["ms_pair"],
                   frac_of_cublas_peak=fl / (res["ms_pair"] * 1e-3) / flops)
        out(res)
    gemm.PAIR = was


def bench_segment(a, out):
    """One prefix layer's attention over a segment: every chunk of the three streams in ONE launch (``dttt_attn_fwd_segment`` /
    ``dttt_attn_bwd_segment``, the clean keys read in place from the window buffer) against one masked call per chunk on
    window keys gathered with ``torch.cat`` (what the layer did before)."""
    from dttt_b200.ops import attention as A, kernels
    B, S, C, W, nh, nkv, d = a.seqs, 3, a.cq, a.window, a.heads, a.kv_heads, a.head_dim
    chunks = a.chunks
    T = chunks * C
    pats = ("full", "full", "causal")
    r = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16)
    q, k, v, g = r(B, S, T, nh, d), r(B, S, T, nkv, d), r(B, S, T, nkv, d), r(B, S, T, nh, d)
    kc = torch.cat([r(B, W * C, nkv, d), k[:, 1]], 1)
    vc = torch.cat([r(B, W * C, nkv, d), v[:, 1]], 1)
    scale = d ** -0.5
    _, flops, src = peaks()
    pairs = 0
    for c in range(chunks):
        nv = A.valid_window_chunks(c + W, W, None)
        pairs += 2 * (nv + 1) * C * C + (nv * C * C + C * (C + 1) // 2)
    fl = 4.0 * B * nh * d * pairs
    fwd = lambda: kernels.attention_fwd_segment(q, kc, vc, k, v, C, W, W, None, pats, scale)
    ms = timeit(fwd, a.iters, a.once)
    o, lse = fwd()
    bwd = lambda: kernels.attention_bwd_segment(g, q, kc, vc, k, v, o, lse, C, W, W, None, pats, scale)
    mb = timeit(bwd, a.iters, a.once)

    def per_chunk(with_bwd):
        for c in range(chunks):
            nv = A.valid_window_chunks(c + W, W, None)
            sl = slice(c * C, (c + 1) * C)
            kw, vw = kc[:, (W + c - nv) * C:(W + c) * C], vc[:, (W + c - nv) * C:(W + c) * C]
            for s_, pat in enumerate(pats):
                oo, ll = kernels.attention_fwd(q[:, s_, sl], kw, vw, scale, pat, k2=k[:, s_, sl], v2=v[:, s_, sl])
                if with_bwd:
                    kernels.attention_bwd(g[:, s_, sl], q[:, s_, sl], kw, vw, oo, ll, scale, pat, k2=k[:, s_, sl], v2=v[:, s_, sl])
    res = {"kernel": "attention, segment form", "seqs": B, "streams": S, "chunks": chunks, "C": C, "W": W, "heads": nh, "kv_heads": nkv,
           "head_dim": d, "ms_fwd": ms, "tflops_fwd": fl / ms / 1e9, "ms_bwd": mb, "tflops_bwd": 2.5 * fl / mb / 1e9,
           "frac_of_cublas_peak_fwd": fl / (ms * 1e-3) / flops, "frac_of_cublas_peak_bwd": 2.5 * fl / (mb * 1e-3) / flops, "peaks": src}
    if a.compare and not a.once:
        m1 = timeit(lambda: per_chunk(False), a.iters)
        m2 = timeit(lambda: per_chunk(True), a.iters)
        res.update(ms_fwd_per_chunk_calls=m1, ms_bwd_per_chunk_calls=m2 - m1, fwd_speedup=m1 / ms, bwd_speedup=(m2 - m1) / mb)
    out(res)


def bench_gdn(a, out):
    """Gated delta rule over one chunk: the blocked WY kernel (``csrc/gdn_chunked.cu``, f32, one CTA per 32 value rows of a head)
    against the same block algebra in PyTorch (batched small GEMMs + triangular solves, differentiated by autograd)."""
    from dttt_b200.ops import gdn_scan, kernels
    B, C, nh, D = a.seqs, a.cq, a.heads, a.head_dim
    gen = torch.Generator(device="cuda").manual_seed(3)
    r = lambda *s: torch.randn(*s, device="cuda", generator=gen)
    k = torch.nn.functional.normalize(r(B, C, nh, D), dim=-1)
    v, beta, la, S0 = r(B, C, nh, D), torch.sigmoid(r(B, C, nh)), -0.05 * torch.rand(B, C, nh, device="cuda", generator=gen), 0.1 * r(B, nh, D, D)
    gS = r(B, nh, D, D)
    hbm, _, src = peaks()
    ms = timeit(lambda: kernels.gdn_chunk_fwd(k, v, beta, la, S0), a.iters, a.once)
    mb = timeit(lambda: kernels.gdn_chunk_bwd(k, v, beta, la, S0, gS), a.iters, a.once)
    fl = B * nh * (C // 64) * 2.0 * (64 * 64 * D + 64 * D * D + 64 * 64 * D + 64 * D * D)        # K K^T, K S^T, solve, U^T K
    res = {"kernel": "gdn_chunk (WY blocks of 64)", "seqs": B, "C": C, "heads": nh, "head_dim": D, "ms_fwd": ms, "ms_bwd": mb,
           "gflops_fwd": fl / ms / 1e6, "peaks": src}
    if a.compare and not a.once:
        was = kernels.gdn_chunk_supported
        kernels.gdn_chunk_supported = lambda *_: False
        try:
            leaves = [t.clone().requires_grad_(True) for t in (k, v, beta, la, S0)]

            def both():
                S = gdn_scan.delta_rule_chunked(*leaves)
                torch.autograd.grad(S, leaves, gS)
            mtb = timeit(both, a.iters)
        finally:
            kernels.gdn_chunk_supported = was
        res.update(ms_fwd_bwd_torch_blocks=mtb, fwd_bwd_speedup_vs_torch=mtb / (ms + mb))
    out(res)


def bench_attn(a, out):
    from dttt_b200.ops import kernels
    n, Cq, Kn, nh, nkv, d = a.seqs, a.cq, a.kn, a.heads, a.kv_heads, a.head_dim
    q = torch.randn(n, Cq, nh, d, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(n, Kn, nkv, d, device="cuda", dtype=torch.bfloat16)
    ms = timeit(lambda: kernels.attention_fwd(q, k, v, d ** -0.5, a.causal, a.variant), a.iters, a.once)
    _, flops, src = peaks()
    pairs = Cq * Kn - (Cq * (Cq - 1) // 2 if a.causal else 0)             # visible (query, key) pairs
    fl = 4.0 * n * nh * d * pairs
    res = {"kernel": "attn_fwd_tcgen05", "seqs": n, "Cq": Cq, "Kn": Kn, "heads": nh, "kv_heads": nkv, "head_dim": d,
           "causal": a.causal, "variant": a.variant, "ms": ms, "tflops": fl / ms / 1e9, "frac_of_cublas_peak": fl / (ms * 1e-3) / flops, "peaks": src}
    if a.compare and not a.once:
        with torch.no_grad():
            mt = timeit(lambda: _sdpa_fast(q, k, v, d ** -0.5, a.causal), a.iters)
        res.update(ms_library=mt, tflops_library=fl / mt / 1e9, vs_library=mt / ms)
    out(res)
    if a.bwd:
        o, lse = kernels.attention_fwd(q, k, v, d ** -0.5, a.causal, a.variant)
        g = torch.randn_like(o)
        mb = timeit(lambda: kernels.attention_bwd(g, q, k, v, o, lse, d ** -0.5, a.causal), a.iters, a.once)
        resb = {"kernel": "attn_bwd_tcgen05", "seqs": n, "Cq": Cq, "Kn": Kn, "heads": nh, "kv_heads": nkv, "head_dim": d,
                "causal": a.causal, "ms": mb, "tflops": 2.5 * fl / mb / 1e9, "frac_of_cublas_peak": 2.5 * fl / (mb * 1e-3) / flops,
                "note": "2.5 x forward FLOPs (five products); includes the delta kernel, the f32 dQ zero-fill and its cast", "peaks": src}
        if a.compare and not a.once:
            qq, kk, vv = (t.detach().requires_grad_(True) for t in (q, k, v))
            oo = _sdpa_fast(qq, kk, vv, d ** -0.5, a.causal)
            ml = timeit(lambda: torch.autograd.grad(oo, (qq, kk, vv), g, retain_graph=True), a.iters)
            resb.update(ms_library=ml, vs_library=ml / mb)
        out(resb)


def bench_attn2(a, out):
    """The derivative of the attention backward (``ops.attn_second``): the row kernel alone against the copy bandwidth, and the
    whole second-order call (4 + 7 tensor-core products around it) against autograd differentiating the staged statement."""
    from dttt_b200.ops import attention, attn_second, kernels
    n, Cq, Kn, nh, nkv, d = a.seqs, a.cq, a.kn, a.heads, a.kv_heads, a.head_dim
    scale = d ** -0.5
    mk = lambda *s: torch.randn(*s, device="cuda", dtype=torch.bfloat16)
    q, k, v, g = mk(n, Cq, nh, d), mk(n, Kn, nkv, d), mk(n, Kn, nkv, d), mk(n, Cq, nh, d)
    cq, ck, cv = mk(n, Cq, nh, d), mk(n, Kn, nkv, d), mk(n, Kn, nkv, d)
    o, lse = kernels.attention_fwd(q, k, v, scale, a.causal)
    hbm, flops, src = peaks()
    rows = n * nh * Cq
    S, dP, gdS, X = (torch.randn(rows, Kn, device="cuda") for _ in range(4))
    lse_r, delta = torch.full((rows,), 8.0, device="cuda"), torch.zeros(rows, device="cuda")
    ms = timeit(lambda: kernels.attention_bwd2_rows(S, dP, gdS, X, lse_r, delta, Cq, a.causal, scale), a.iters, a.once)
    nbytes = rows * Kn * 24.0
    out({"kernel": "attn_bwd2_rows", "rows": rows, "Kn": Kn, "causal": a.causal, "ms": ms, "gbs": nbytes / ms / 1e6,
         "frac_of_copy_bw": nbytes / (ms * 1e-3) / hbm, "note": "4 f32 reads + 4 bf16 writes per score", "peaks": src})
    del S, dP, gdS, X
    if a.compare and not a.once:                      # the products around the row kernel, one of each kind
        from dttt_b200.ops.gemm import gemm_raw
        B, R = n * nkv, (nh // nkv) * Cq
        qg, kg = mk(B, R, d), mk(B, Kn, d)
        q2, k2 = mk(B, R, 2 * d), mk(B, Kn, 2 * d)
        Pm = mk(B, R, Kn)
        acc_r, acc_k = torch.zeros(B, R, d, device="cuda"), torch.zeros(B, Kn, d, device="cuda")
        for name, fn, nb in (("scores f32 = q k^T", lambda: gemm_raw(qg, kg, False, True, torch.float32), B * R * Kn * 4.0),
                             ("scores f32, inner 128", lambda: gemm_raw(q2, k2, False, True, torch.float32), B * R * Kn * 4.0),
                             ("row side: P @ k (f32 accumulate)", lambda: gemm_raw(Pm, kg, False, False, torch.float32, out=acc_r, accumulate=True), B * R * Kn * 2.0),
                             ("key side: P^T @ q (f32 accumulate)", lambda: gemm_raw(Pm, qg, True, False, torch.float32, out=acc_k, accumulate=True), B * R * Kn * 2.0)):
            t = timeit(fn, a.iters)
            out({"kernel": "attn_second_order product: " + name, "batch": B, "rows": R, "Kn": Kn, "ms": t, "gbs": nb / t / 1e6,
                 "frac_of_copy_bw": nb / (t * 1e-3) / hbm, "peaks": src})
        del Pm
    if kernels.available("attention_bwd2_scores") and kernels.attention_bwd2_scores_supported(q, k):
        dl = torch.zeros(n, nh, Cq, device="cuda")
        ms = timeit(lambda: kernels.attention_bwd2_scores(q, g, cq, k, v, ck, cv, lse, dl, scale, a.causal), a.iters, a.once)
        fl5 = 2.0 * n * nh * d * Cq * Kn * 5 * 2                          # five products, two sweeps
        out({"kernel": "attn_bwd2_scores_tcgen05", "seqs": n, "Cq": Cq, "Kn": Kn, "heads": nh, "causal": a.causal, "ms": ms,
             "tflops": fl5 / ms / 1e9, "write_gbs": rows * Kn * 8.0 / ms / 1e6, "frac_of_copy_bw": rows * Kn * 8.0 / (ms * 1e-3) / hbm,
             "note": "replaces the four f32 score products and the row kernel; 8 bytes written per score", "peaks": src})
    ms2 = timeit(lambda: attn_second.second_order(cq, ck, cv, g, q, k, v, o, lse, scale, a.causal), a.iters, a.once)
    pairs = Cq * Kn
    fl = 2.0 * n * nh * d * pairs * 12                                   # 5 score-shaped + 7 output products, dense
    res = {"kernel": "attn_second_order (GEMMs + row kernel)", "seqs": n, "Cq": Cq, "Kn": Kn, "heads": nh, "kv_heads": nkv, "head_dim": d,
           "causal": a.causal, "ms": ms2, "tflops_dense": fl / ms2 / 1e9, "min_bytes_ms": rows * Kn * 54.0 / hbm * 1e3, "peaks": src}
    if a.compare and not a.once:
        def by_autograd():
            ins = [t.detach().requires_grad_(True) for t in (q, k, v)]
            gg = g.detach().requires_grad_(True)
            oo = attention._ref_for_staged(*ins, scale, a.causal)
            first = torch.autograd.grad(oo, ins, gg, create_graph=True)
            L = sum((c.float() * f.float()).sum() for c, f in zip((cq, ck, cv), first))
            return torch.autograd.grad(L, ins + [gg])
        mr = timeit(by_autograd, max(3, a.iters // 3))
        res.update(ms_autograd_of_statement=mr, vs_autograd=mr / ms2,
                   note="the autograd figure includes the statement's forward and first backward, which the kernel path replaces by the flash kernels")
    out(res)


def bench_ce(a, out):
    """Linear + cross-entropy: the forward (GEMM with the per-tile softmax-partials epilogue + combine) and one vocabulary
    block of the backward's dlogits GEMM, against the unfused statement (f32 logits GEMM + torch logsumexp)."""
    from dttt_b200.ops import gemm, kernels
    N, K, V = a.rows, a.k, a.vocab
    h = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    E = (torch.randn(V, K, device="cuda") * 0.02).to(torch.bfloat16)
    y = torch.randint(0, V, (N,), device="cuda")
    _, flops, src = peaks()
    ms = timeit(lambda: kernels.linear_ce_fwd(h, E, y), a.iters, a.once)
    fl = 2.0 * N * K * V
    res = {"kernel": "linear_ce_fwd (gemm_bf16_kernel<256,1> + ce_combine)", "rows": N, "K": K, "classes": V, "ms": ms,
           "tflops": fl / ms / 1e9, "frac_of_cublas_peak": fl / (ms * 1e-3) / flops, "peaks": src}
    if a.compare and not a.once:
        def unfused():
            lg = gemm.gemm_raw(h, E, False, True, torch.float32)
            return torch.logsumexp(lg, -1) - lg.gather(1, y[:, None]).squeeze(1)
        mt = timeit(unfused, a.iters)
        res.update(ms_unfused=mt, vs_unfused=mt / ms)
    out(res)
    lse, _ = kernels.linear_ce_fwd(h, E, y)
    coef = torch.rand(N, device="cuda")
    blk = min(8192, V)
    yi = y.to(torch.int32)
    ms = timeit(lambda: kernels.linear_ce_dlogits(h, E[:blk], yi, coef, lse, 0), a.iters, a.once)
    fl = 2.0 * N * K * blk
    out({"kernel": "linear_ce_dlogits (gemm_bf16_kernel<256,2>)", "rows": N, "K": K, "classes_block": blk, "ms": ms, "tflops": fl / ms / 1e9,
         "frac_of_cublas_peak": fl / (ms * 1e-3) / flops, "peaks": src})


def main(argv=None):
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.kernel_bench")
    ap.add_argument("cmd", choices=["gemm", "gemm_forms", "gemm_pair", "attn", "attn2", "segment", "gdn", "ce", "rmsnorm", "rope", "swiglu", "adamw", "suite"])
    ap.add_argument("--seqs", type=int, default=8); ap.add_argument("--cq", type=int, default=1024); ap.add_argument("--kn", type=int, default=9216)
    ap.add_argument("--heads", type=int, default=32); ap.add_argument("--kv-heads", type=int, default=8); ap.add_argument("--head-dim", type=int, default=64)
    ap.add_argument("--vocab", type=int, default=128256); ap.add_argument("--causal", action="store_true"); ap.add_argument("--variant", type=int, default=0); ap.add_argument("--bwd", action="store_true")
    ap.add_argument("--m", type=int, default=8192); ap.add_argument("--n", type=int, default=8192); ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--batch", type=int, default=1); ap.add_argument("--ta", action="store_true"); ap.add_argument("--tb", action="store_true")
    ap.add_argument("--f32acc", action="store_true"); ap.add_argument("--compare", action="store_true")
    ap.add_argument("--rows", type=int, default=49152); ap.add_argument("--dim", type=int, default=2048)
    ap.add_argument("--iters", type=int, default=10); ap.add_argument("--once", action="store_true")
    ap.add_argument("--window", type=int, default=8, help="segment: window chunks"); ap.add_argument("--chunks", type=int, default=8, help="segment: chunks per segment")
    ap.add_argument("--out", default="")
    ap.add_argument("--tile-form", type=int, default=-1, help="plain GEMM tile form: -1 per shape, 0 128 x 256, 1 256 x 256")
    a = ap.parse_args(argv)
    sys.path.insert(0, ROOT)
    if a.tile_form != -1:
        from dttt_b200.ops import gemm as _g
        _g.set_tile_form(a.tile_form)
    lines = []

    def out(d):
        lines.append(json.dumps(d))
        print(lines[-1], flush=True)
    if a.cmd == "gemm":
        bench_gemm(a, out)
    elif a.cmd == "attn":
        bench_attn(a, out)
    elif a.cmd == "gemm_forms":
        bench_gemm_forms(a, out)
    elif a.cmd == "gemm_pair":
        bench_gemm_pair(a, out)
    elif a.cmd == "segment":
        bench_segment(a, out)
    elif a.cmd == "gdn":
        a.heads = 16 if a.heads == 32 else a.heads
        a.head_dim = 128 if a.head_dim == 64 else a.head_dim
        bench_gdn(a, out)
    elif a.cmd == "attn2":
        bench_attn2(a, out)
    elif a.cmd == "ce":
        a.rows = 2048 if a.rows == 49152 else a.rows
        a.k = 2048 if a.k == 8192 else a.k
        bench_ce(a, out)
    elif a.cmd == "suite":
        a.compare = True
        shapes = [(8192, 8192, 8192, 1, 0, 0, 0), (49152, 2048, 2048, 1, 0, 0, 0), (49152, 8192, 2048, 1, 0, 0, 0), (49152, 2048, 8192, 1, 0, 0, 0),
                  (2048, 8192, 2048, 1, 0, 0, 0), (2048, 2048, 8192, 1, 0, 0, 0), (1024, 8192, 2048, 4, 0, 0, 0), (2048, 8192, 1024, 4, 1, 0, 0),
                  (2048, 8192, 49152, 1, 1, 0, 1), (49152, 2048, 8192, 1, 0, 1, 0), (2048, 8192, 2048, 1, 0, 1, 0), (8192, 2048, 2048, 1, 1, 0, 1)]
        for M, N, K, B, ta, tb, acc in shapes:
            a.m, a.n, a.k, a.batch, a.ta, a.tb, a.f32acc = M, N, K, B, bool(ta), bool(tb), bool(acc)
            bench_gemm(a, out)
        for n, Cq, Kn, causal in ((8, 1024, 9216, True), (8, 1024, 9216, False), (16, 1024, 1024, True), (8, 1024, 4096, True)):
            a.seqs, a.cq, a.kn, a.causal, a.heads, a.kv_heads, a.head_dim, a.bwd = n, Cq, Kn, causal, 32, 8, 64, True
            bench_attn(a, out)
        a.seqs, a.cq, a.kn, a.causal, a.heads, a.kv_heads, a.head_dim = 8, 1024, 9216, True, 16, 4, 128
        bench_attn(a, out)
        bench_gemm_pair(a, out)
        a.seqs, a.cq, a.heads, a.kv_heads, a.head_dim, a.window, a.chunks = 2, 1024, 32, 8, 64, 7, 8
        bench_segment(a, out)
        a.seqs, a.cq, a.heads, a.head_dim = 4, 1024, 16, 128
        bench_gdn(a, out)
        a.rows, a.k, a.vocab = 2048, 2048, 128256
        bench_ce(a, out)
        for cmd, R, D in (("rmsnorm", 49152, 2048), ("swiglu", 49152, 8192), ("rope", 49152, 2048), ("adamw", 16384, 8192)):
            a.cmd, a.rows, a.dim = cmd, R, D
            bench_elementwise(a, out)
    else:
        bench_elementwise(a, out)
    if a.out:
        with open(a.out, "w") as fh:
            fh.write("\n".join(lines) + "\n")


if __name__ == "__main__":
    main()
