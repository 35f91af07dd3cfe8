// Shared by the attention kernels: own-chunk patterns as per-row key intervals, and the geometry of the segment form.
#pragma once
#include <cuda_runtime.h>

namespace dttt {

// Own-chunk patterns (reference src/ttt/attention.py:132-159).  For every pattern the keys a query row sees are a prefix
// [0, e1] of the key axis plus, for the sub-block read only, one more interval [s2, e2]; the key axis is
// [window | (clean own keys, read only) | own keys] and `i` is the query's slot in its chunk.
enum : int { MASK_FULL = 0, MASK_CAUSAL = 1, MASK_SPLIT = 2, MASK_BLOCK = 3, MASK_READ = 4 };
constexpr int MAX_STREAMS = 8;
constexpr float MASKED = -3.0e38f;   // below the running maximum's initial value, so a fully masked block leaves it alone

struct RowMask { int e1, s2, e2; };

__device__ __forceinline__ RowMask row_mask(int mode, int param, int i, int Kn, int Cq) {
  const int own = Kn - Cq;
  RowMask r;
  r.s2 = 1; r.e2 = 0;                                                     // empty
  switch (mode) {
    case MASK_CAUSAL: r.e1 = own + i; break;
    case MASK_SPLIT:  r.e1 = own + max(i, param - 1); break;              // the first `param` keys, then causal
    case MASK_BLOCK:  r.e1 = own + (i / param + 1) * param - 1; break;    // own sub-block and the earlier ones
    case MASK_READ:                                                       // clean keys of earlier sub-blocks, noisy keys of the own one
      r.e1 = own - Cq + (i / param) * param - 1;
      r.s2 = own + (i / param) * param;
      r.e2 = min(r.s2 + param - 1, Kn - 1);
      break;
    default: r.e1 = Kn - 1;
  }
  r.e1 = min(r.e1, Kn - 1);
  return r;
}


// Segment form: "sequence" v = (b, stream s, chunk c) of a [B, streams, chunks * C] layout.  Its window keys are rows
// [(W + c - nv) C, (W + c) C) of the clean stream's [previous window | segment] buffer of sequence b (no copy of the windows is
// ever made), its own keys chunk c of stream s; nv = min(first + c, W, reach) window chunks are visible.
struct SegSpec {
  int on, streams, chunks, first, W, reach;
  int mode[MAX_STREAMS], param[MAX_STREAMS];
};

// What one (virtual) sequence of a launch reads: Kn keys of which the first Kn1 come from the first key / value tensor (rows
// row0 ... of its sequence kb), the rest from the second; own-chunk pattern (mode, param); nv window chunks.
struct SeqGeom {
  int Kn, Kn1, mode, param, kb, row0, nv, stream, chunk;
};

__host__ __device__ __forceinline__ int seg_visible_chunks(const SegSpec& sg, int c) {
  int nv = sg.first + c < sg.W ? sg.first + c : sg.W;
  if (sg.reach >= 0 && sg.reach < nv) nv = sg.reach;
  return nv;
}

__device__ __forceinline__ SeqGeom seq_geom(const SegSpec& sg, int v, int C, int Kn, int Kn1, int mode, int param) {
  SeqGeom g;
  if (!sg.on) {
    g.Kn = Kn; g.Kn1 = Kn1; g.mode = mode; g.param = param; g.kb = v; g.row0 = 0; g.nv = 0; g.stream = 0; g.chunk = 0;
    return g;
  }
  const int per_b = sg.streams * sg.chunks;
  g.chunk = v % sg.chunks;
  g.stream = (v / sg.chunks) % sg.streams;
  g.nv = seg_visible_chunks(sg, g.chunk);
  g.mode = sg.mode[g.stream]; g.param = sg.param[g.stream];
  g.kb = v / per_b;
  g.row0 = (sg.W + g.chunk - g.nv) * C;
  g.Kn1 = g.nv * C + (g.mode == MASK_READ ? C : 0);          // the clean own chunk follows the window in the same buffer
  g.Kn = g.Kn1 + C;
  return g;
}

}  // namespace dttt
