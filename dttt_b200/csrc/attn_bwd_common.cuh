// Shared by the attention backward kernels (head dimension 64 and 128): parameters, TMA helpers, and the part of a CTA's
// start-up that does not depend on the head dimension: which key block the CTA owns and the list of (sequence, query tile)
// work items that see it.
#pragma once
#include "ptx_sm100.cuh"
#include "attn_common.cuh"

namespace dttt {

constexpr int BQ = 128, BKEY = 128;
constexpr int MAX_ITEMS = 512;


struct AttnBwdParams {
  int n, Cq, Kn, nh, nkv, causal;
  int Kn1;              // keys [0, Kn1) belong to the first K / V pair (and dK / dV), the rest to the second
  int mask_mode, mask_param;
  SegSpec sg;           // segment form: dK / dV mirror the clean buffer [B, (W + chunks) C, nkv, d], dK2 / dV2 the streams' own keys
  float scale;
  const float* lse;     // [n, nh, Cq]
  const float* delta;   // [n, nh, Cq]  rowsum(dO * O)
  float* dQ;            // [n, Cq, nh, d] f32, accumulated into
  __nv_bfloat16* dK;    // [n, Kn1, nkv, d]
  __nv_bfloat16* dV;
  __nv_bfloat16* dK2;   // [n, Kn - Kn1, nkv, d]
  __nv_bfloat16* dV2;
  int* status;
};

__device__ __forceinline__ void tma_load_4d_b(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// Barrier `id` over `nthreads` threads that also ANDs a per-thread flag: every participant gets the same verdict.
__device__ __forceinline__ int bar_red_and(int id, int nthreads, int flag) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, %2, %3, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(out) : "r"(flag), "r"(id), "r"(nthreads) : "memory");
  return out;
}

// dst[tile] += smem tile, as one bulk tensor reduction (f32 add) issued by a single thread
__device__ __forceinline__ void tma_reduce_add_4d(const CUtensorMap* map, const void* smem_src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.reduce.async.bulk.tensor.4d.global.shared::cta.add.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void bar_sync_named(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }


// The key block a CTA owns: which tensor pair it lies in, its sequence and first row there, and the rows per sequence of
// that tensor (for the output offset).  `live` is false for grid cells beyond the tensor's end.
struct OwnedBlock {
  bool live, second;
  int kseq, krow, klen;
};

__device__ __forceinline__ OwnedBlock owned_block(const AttnBwdParams& p, int jb, int z) {
  OwnedBlock o;
  if (!p.sg.on) {
    o.live = jb * BKEY < p.Kn;
    o.second = jb * BKEY >= p.Kn1;
    o.kseq = z;
    o.krow = o.second ? jb * BKEY - p.Kn1 : jb * BKEY;
    o.klen = o.second ? p.Kn - p.Kn1 : p.Kn1;
  } else {
    // z = (sequence, stream): the clean stream's CTAs walk the clean buffer, the others their own keys
    const int bb = z / p.sg.streams, st = z % p.sg.streams;
    o.second = st != 1;
    o.klen = o.second ? p.sg.chunks * p.Cq : (p.sg.W + p.sg.chunks) * p.Cq;
    o.live = jb * BKEY < o.klen;
    o.krow = jb * BKEY;
    o.kseq = o.second ? z : bb;                              // own keys are [B * streams, chunks * C]; the clean buffer [B, ...]
  }
  return o;
}

// Fills `items` with every (sequence, query tile) that sees at least one key of the block: .x = sequence, .y = query tile * 2 +
// needs-mask + (stream << 24), .z = position of the block's first key on that sequence's key axis, .w = that sequence's number of
// keys (what the math warps need for the mask, so that no step recomputes the geometry).  Returns how many there are (which
// may exceed MAX_ITEMS: the caller reports that).  One thread runs this.
__device__ inline int build_work_items(const AttnBwdParams& p, const OwnedBlock& o, int jb, int z, int4* items) {
  const int nqt = (p.Cq + BQ - 1) / BQ;
  int n = 0;
  auto consider = [&](int v, const SeqGeom& G, int kpos0) {
    // key block = positions [kpos0, kpos0 + 127] of sequence v's key axis
    for (int qt = 0; qt < nqt; ++qt) {
      const int i0 = qt * BQ, i1 = min(i0 + BQ - 1, p.Cq - 1);
      const RowMask a = row_mask(G.mode, G.param, i0, G.Kn, p.Cq), zz = row_mask(G.mode, G.param, i1, G.Kn, p.Cq);
      const bool any = (kpos0 <= zz.e1) || (kpos0 + BKEY - 1 >= a.s2 && kpos0 <= zz.e2);
      if (!any) continue;
      const bool all = (kpos0 + BKEY - 1 <= a.e1) || (kpos0 >= zz.s2 && kpos0 + BKEY - 1 <= a.e2);
      const bool ragged = kpos0 + BKEY > G.Kn;
      if (n < MAX_ITEMS) items[n] = make_int4(v, qt * 2 + ((all && !ragged) ? 0 : 1) + (G.stream << 24), kpos0, G.Kn);
      ++n;
    }
  };
  if (!p.sg.on) {
    const SeqGeom G = seq_geom(p.sg, z, p.Cq, p.Kn, p.Kn1, p.mask_mode, p.mask_param);
    consider(z, G, jb * BKEY);
    return n;
  }
  const int bb = z / p.sg.streams, st = z % p.sg.streams;
  const int per_b = p.sg.streams * p.sg.chunks;
  if (o.second) {
    const int c = o.krow / p.Cq;
    const int v = bb * per_b + st * p.sg.chunks + c;
    const SeqGeom G = seq_geom(p.sg, v, p.Cq, 0, 0, 0, 0);
    consider(v, G, G.Kn - p.Cq + (o.krow - c * p.Cq));
    return n;
  }
  // a block of the clean buffer: row krow = chunk (krow / C - W) of the segment (negative: the previous segment's window)
  const int kc = o.krow / p.Cq - p.sg.W;
  for (int c = max(kc, 0); c < min(kc + p.sg.W + 1, p.sg.chunks); ++c)
    for (int s2 = 0; s2 < p.sg.streams; ++s2) {
      const int v = bb * per_b + s2 * p.sg.chunks + c;
      const SeqGeom G = seq_geom(p.sg, v, p.Cq, 0, 0, 0, 0);
      const int kpos0 = o.krow - G.row0;
      // the stream reads this buffer up to its window (nv chunks), the clean stream (and a reading stream) one chunk further
      const int reach_rows = G.nv * p.Cq + ((s2 == 1 || G.mode == MASK_READ) ? p.Cq : 0);
      if (kpos0 < 0 || kpos0 >= reach_rows) continue;
      consider(v, G, kpos0);
    }
  return n;
}

// The visible keys of query row `qi` of a work item, as positions relative to the owned block's first row.
__device__ __forceinline__ RowMask item_row_mask(const AttnBwdParams& p, const int4& item, int qi) {
  const int stream = item.y >> 24;
  const int mode = p.sg.on ? p.sg.mode[stream] : p.mask_mode, param = p.sg.on ? p.sg.param[stream] : p.mask_param;
  RowMask rm = row_mask(mode, param, min(qi, p.Cq - 1), item.w, p.Cq);
  rm.e1 -= item.z; rm.s2 -= item.z; rm.e2 -= item.z;
  return rm;
}
__device__ __forceinline__ int item_qt(const int4& item) { return (item.y & 0xffffff) >> 1; }

}  // namespace dttt
