"""Analytic per-GPU memory, FLOP and MFU model of a training step on B200.

    python -m dttt_b200.tools.memory_model --config configs/b200_1b_8k --seq_len 8192 --seqs_per_gpu 2 --gpus 8 [--step_time S]

Parameters, the per-sequence memory carried through the chunk pass (f32 fast weight + suffix KV window), the
persistent state under the sharding of ``parallel.store`` (f32 master + two moments split over FSDP; full bf16
compute copy and full f32 gradient buffer per GPU), what the recompute regions keep, and the model FLOPs per token
(matmuls only: what MFU counts) next to the hardware FLOPs including recomputation.  The FLOP accounting follows
the reference's ``tools/memory_model.py:70-101``: per chunk the suffix runs forwards A, B, C, the inner backward of
C and the outer backward through all of it (second order); the prefix runs three streams forward and backward;
window attention costs ``4 * keys * nh * d`` per token and layer.
"""
from __future__ import annotations

import argparse
import json
import math
import os

GIB = 1024 ** 3
HBM_GIB = 180.0


def _cfg(path: str) -> dict:
    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as fh:
        c = json.load(fh)
    c.setdefault("ttt_intermediate_size", None)
    c.setdefault("suffix_plain_top", 0)
    return c


def params(c: dict) -> dict:
    H, I, L, S = c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"], c["suffix_len"]
    nh, nkv, d = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"]
    F = S - c.get("suffix_plain_top", 0) if not c.get("fast_layers") else len(c["fast_layers"])
    attn = H * nh * d + 2 * H * nkv * d + nh * d * H + (2 * d if c.get("qk_norm", True) else 0)
    mlp = 3 * H * I
    Ip = c["ttt_intermediate_size"] or I
    emb = c["vocab_size"] * H * (1 if c.get("tie_word_embeddings", True) else 2)
    base = L * (attn + mlp + 2 * H) + H
    prime = F * (3 * H * Ip + 2 * H) if c.get("memory", "ttt") == "ttt" else 0
    return {"attn_per_layer": attn, "mlp_per_layer": mlp, "base": base, "prime": prime, "embed": emb, "total": base + prime + emb, "fast_layers": F}


def carry_bytes(c: dict) -> dict:
    H, S = c["hidden_size"], c["suffix_len"]
    Ip = c["ttt_intermediate_size"] or c["intermediate_size"]
    F = params(c)["fast_layers"]
    win = c.get("window_chunks", 1) * c["chunk_size"]
    if c.get("memory", "ttt") == "gdn":
        fw = S * c.get("gdn_heads", 16) * c.get("gdn_head_dim", 128) ** 2 * 4
    else:
        fw = F * 3 * H * Ip * 4
    return {"fast_weight": fw, "kv": S * win * 2 * c["num_key_value_heads"] * c["head_dim"] * 2}


def flops_per_token(c: dict, seq_len: int, keep_prefix_layers: int = 0, keep_suffix_chunks: int = 0, segment_chunks: int = 0) -> tuple:
    """``(model, hardware)`` FLOPs per token of one training step.  Prefix layers / chunk steps that keep their graph
    (``keep_prefix_layers`` / ``keep_suffix_chunks`` per segment) are not recomputed."""
    H, I, L, S = c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"], c["suffix_len"]
    nh, nkv, d, C, W, V = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], c["chunk_size"], c["window_chunks"], c["vocab_size"]
    Ip = c["ttt_intermediate_size"] or I
    nc = seq_len // C
    p_layer = H * nh * d + 2 * H * nkv * d + nh * d * H + 3 * H * I
    p_prime = 3 * H * Ip if c.get("memory", "ttt") == "ttt" else 0
    keys = sum(min(i, W) + 1 for i in range(nc)) / nc * C                 # invalid window chunks are never computed
    attn = 4 * keys * nh * d
    fwd_prefix = (L - S) * (2 * p_layer + attn)
    fwd_suffix = S * (2 * (p_layer + p_prime) + attn)
    ce = 2 * V * H
    model = (3 * fwd_prefix * 3 + 3 * fwd_suffix + 2 * ce + 2 * (fwd_suffix + ce)
             + 2 * (2 * fwd_suffix + ce + 3 * (fwd_suffix + ce)))
    per_seg = segment_chunks or nc
    frac_suffix = 1.0 - min(keep_suffix_chunks, per_seg) / per_seg
    frac_prefix = 1.0 - min(keep_prefix_layers, L - S) / max(1, L - S)
    # one recompute of each region that is not kept
    hardware = model + frac_suffix * (3 * fwd_suffix + 2 * ce + 2 * (fwd_suffix + ce)) + frac_prefix * 3 * fwd_prefix
    return model, hardware


def kept_bytes(c: dict, seq_len: int, keep_prefix_layers: int, keep_suffix_chunks: int, segment_chunks: int = 0) -> float:
    """Bytes per sequence of the graphs that stay resident.  Per token a kept prefix layer holds about ``5 H + 3 I`` bf16 values for
    each of the three streams; a kept chunk step about ``3.75 (5 H + 3 I + 3 I')`` per suffix layer (streams A and B at first
    order, the recorded inner stream C).  Both factors are fitted to measurements of the 1B model at 8k on a B200 (3.45 GB per
    kept prefix layer and 3.65 GB per kept chunk step, for two sequences)."""
    H, I, L, S, C = c["hidden_size"], c["intermediate_size"], c["num_hidden_layers"], c["suffix_len"], c["chunk_size"]
    Ip = (c["ttt_intermediate_size"] or I) if c.get("memory", "ttt") == "ttt" else 0
    nc = seq_len // C
    per_seg = segment_chunks or nc
    kept_chunks = (nc // per_seg) * min(keep_suffix_chunks, per_seg)
    prefix = min(keep_prefix_layers, L - S) * 3 * seq_len * (5 * H + 3 * I) * 2
    suffix = kept_chunks * C * S * 3.75 * (5 * H + 3 * I + 3 * Ip) * 2
    return prefix + suffix


def report(c: dict, seq_len: int, seqs_per_gpu: int, gpus: int, fsdp: int, step_time: float = 0.0, micro: int = 0,
           keep_prefix_layers: int = 0, keep_suffix_chunks: int = 0, segment_chunks: int = 0) -> dict:
    p = params(c)
    k = carry_bytes(c)
    micro = micro or seqs_per_gpu
    nc = seq_len // c["chunk_size"]
    H, L, S = c["hidden_size"], c["num_hidden_layers"], c["suffix_len"]
    persistent = p["total"] * (12 / fsdp + 2 + 4)                          # sharded f32 master+moments, full bf16 copy, full f32 grads
    regions = micro * ((L - S) * 3 * seq_len * H * 2 + nc * (k["fast_weight"] + k["kv"]))
    model, hw = flops_per_token(c, seq_len, keep_prefix_layers, keep_suffix_chunks, segment_chunks)
    kept = micro * kept_bytes(c, seq_len, keep_prefix_layers, keep_suffix_chunks, segment_chunks)
    out = {"params": p, "kept_graphs_gib": kept / GIB, "carry_gib_per_seq": (k["fast_weight"] + k["kv"]) / GIB, "persistent_gib": persistent / GIB,
           "region_inputs_gib": regions / GIB, "model_gflop_per_token": model / 1e9, "hardware_gflop_per_token": hw / 1e9,
           "dense_6n_gflop_per_token": 6 * p["total"] / 1e9,
           "drift_bound_per_chunk": 1.0 / (c.get("initializer_range", 0.02) * math.sqrt(max(1, p["prime"])))}
    if step_time > 0:
        peaks = os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "MEASURED_PEAKS.json")
        peak = json.load(open(peaks))["bf16_tflops_sustained"] * 1e12 if os.path.exists(peaks) else 1.4e15
        tok = seqs_per_gpu * seq_len
        out.update(tokens_per_s_per_gpu=tok / step_time, model_tflops_per_gpu=model * tok / step_time / 1e12,
                   mfu_of_sustained_cublas=model * tok / step_time / peak, hardware_frac=hw * tok / step_time / peak)
    return out


def main(argv=None) -> None:
    ap = argparse.ArgumentParser(prog="python -m dttt_b200.tools.memory_model")
    ap.add_argument("--config", default="configs/b200_1b_8k")
    ap.add_argument("--seq_len", type=int, default=8192)
    ap.add_argument("--seqs_per_gpu", type=int, default=2)
    ap.add_argument("--micro", type=int, default=0)
    ap.add_argument("--gpus", type=int, default=8)
    ap.add_argument("--fsdp", type=int, default=0)
    ap.add_argument("--step_time", type=float, default=0.0)
    ap.add_argument("--keep_prefix_layers", type=int, default=0)
    ap.add_argument("--keep_suffix_chunks", type=int, default=0)
    ap.add_argument("--segment_chunks", type=int, default=0)
    a = ap.parse_args(argv)
    c = _cfg(a.config)
    r = report(c, a.seq_len, a.seqs_per_gpu, a.gpus, a.fsdp or a.gpus, a.step_time, a.micro, a.keep_prefix_layers, a.keep_suffix_chunks,
               a.segment_chunks)
    p = r["params"]
    print(f"=== {a.config} @ {a.seq_len} ===")
    print(f"  parameters: base {p['base'] / 1e6:.1f} M  fast weight {p['prime'] / 1e6:.1f} M  embedding {p['embed'] / 1e6:.1f} M  total {p['total'] / 1e9:.4f} B")
    print(f"  carried per sequence: {r['carry_gib_per_seq']:.3f} GiB (f32 fast weight + suffix KV window)")
    print(f"  per GPU: persistent {r['persistent_gib']:.1f} GiB + region inputs {r['region_inputs_gib']:.1f} GiB + kept graphs "
          f"{r['kept_graphs_gib']:.1f} GiB of {HBM_GIB:.0f} GiB (transients of the pass in flight come on top)")
    print(f"  FLOPs per token: model {r['model_gflop_per_token']:.1f} G, hardware incl. recompute {r['hardware_gflop_per_token']:.1f} G "
          f"({r['dense_6n_gflop_per_token']:.1f} G for a dense LM of the same size)")
    if a.step_time:
        print(f"  {r['tokens_per_s_per_gpu']:.0f} tok/s/GPU = {r['model_tflops_per_gpu']:.0f} model TFLOP/s/GPU = "
              f"{100 * r['mfu_of_sustained_cublas']:.1f}% of sustained cuBLAS bf16 (hardware {100 * r['hardware_frac']:.1f}%)")


if __name__ == "__main__":
    main()
