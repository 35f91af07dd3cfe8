// Chunk-window flash attention, backward, on tcgen05 tensor cores (head dimension 64).
//
// Given Q, K, V, O, dO and the forward's LSE (layouts of attn_fwd_tcgen05.cu) this produces dQ, dK, dV of
//   O = softmax(scale * Q K^T + mask) V        (reference src/ttt/attention.py:181-201, first-order VJP).
//
// One CTA owns one block of 128 keys of one (sequence, KV head) and walks over every query tile that sees it,
// for each of the rep = nh / nkv query heads of the group; dK and dV of the block accumulate in tensor memory over
// the whole walk (so GQA needs no atomics for them), dQ tiles are produced per step and added into an f32 buffer.
// Everything is computed transposed (keys on TMEM lanes, queries on columns) so that P^T and dS^T, written back to
// tensor memory as bf16 pairs by the thread that owns the key row, are directly the A operands of
//   dV += P^T dO      dK += dS^T Q                      (A from TMEM)
// and dS^T, also written to shared memory, is the M-major A operand of  dQ = dS K.
// Per step:   S^T = K Q^T,  dP^T = V dO^T   ->   P^T = exp2(S^T sl2 - LSE),  dS^T = P^T (dP^T - D) scale.
// A step works on its 128 queries as two halves of 64: while the warps do the elementwise work of one half the tensor
// core runs dV / dK of the other half and already the S^T / dP^T of the next step's first half (the TMEM columns of a
// half are free as soon as its dV / dK products have been issued; the tensor pipe runs its queue in order).  The dQ
// tile of a step is reduced into global memory during the next step, and dS^T alternates between two shared-memory
// tiles so that the next step may overwrite one while dQ still reads the other.
//
//   warp 0      TMA: K, V once; Q and dO tiles into two stages
//   warp 1      tcgen05.mma issuer, TMEM owner
//   warps 2-9   two per TMEM lane quarter: softmax-backward math, then the step's dQ tile goes through shared memory
//               into global memory by bulk tensor reductions (cp.reduce.async.bulk.tensor, f32 add), then the
//               final dK / dV stores
//   warps 10-17 (the default, sixteen-warp form) a second group of eight: group h owns the 64-query half h of every step and
//               the 32-column half h of the dQ tile, so the elementwise work of both halves runs at the same time
// TMEM columns: S^T / P^T [0,128)  dP^T / dS^T [128,256)  dV [256,320)  dK [320,384)  dQ [384,448).
// Every wait is bounded (ptx_sm100.cuh); on a timeout the roles leave through the common exit and TMEM is freed.
//
// Which queries a key block meets is a LIST of work items built when the CTA starts: (sequence, query tile) pairs that see
// at least one key of the block under the own-chunk pattern (attn_common.cuh).  In the plain form the list holds the query
// tiles of the block's own sequence.  In the segment form a block of the clean stream's [previous window | segment] buffer
// is met by every stream's chunks that have it in their window and by the clean stream's own chunk, so the gradient of a
// clean key is accumulated once, in tensor memory, over all of them (no per-window partial gradients to add up afterwards).
#include "attn_bwd_common.cuh"
#include "host_check.h"

#include <mutex>
#include <cstring>
#include <cstdlib>

namespace dttt {

constexpr int HD = 64;

struct BwdSmem {
  static constexpr int TILE = 128 * HD * 2;                 // 16 KB: one [128, 64] bf16 tile
  static constexpr int DS_BYTES = 128 * 128 * 2;            // dS^T for the dQ product
  static constexpr int STAGES = 2;
  static constexpr int AUX = 2 * 2 * 128 * 4;               // LSE and D, two buffers
  static constexpr int DQ_BYTES = 128 * HD * 4;                // f32 dQ tile staged for the bulk reduction
  static constexpr int MASK = 2 * 3 * 128 * 4;              // per query column: e1, s2, e2 (two buffers)
  static constexpr int ITEMS = MAX_ITEMS * 16;              // work items (build_work_items)
  static constexpr int TOTAL = 2 * TILE + STAGES * 2 * TILE + 2 * DS_BYTES + DQ_BYTES + AUX + MASK + ITEMS + 1024 + 1024;
};

// delta[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d]; eight threads per row of 64.
__global__ void attn_bwd_delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO,
                                      float* __restrict__ delta, long long rows, int Cq, int nh) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid >> 3;                            // row = (b * Cq + i) * nh + h
  const int part = (int)(gid & 7);
  float acc = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(O + row * HD + part * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(dO + row * HD + part * 8);
    const __nv_bfloat162* ab = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&g);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 x = __bfloat1622float2(ab[q]), y = __bfloat1622float2(gb[q]);
      acc += x.x * y.x + x.y * y.y;
    }
  }
  acc += __shfl_xor_sync(0xffffffffu, acc, 1);
  acc += __shfl_xor_sync(0xffffffffu, acc, 2);
  acc += __shfl_xor_sync(0xffffffffu, acc, 4);
  if (part == 0 && row < rows) {
    const long long bi = row / nh;                           // b * Cq + i
    const int h = (int)(row - bi * nh);
    const long long b = bi / Cq;
    const int i = (int)(bi - b * Cq);
    delta[(b * nh + h) * Cq + i] = acc;
  }
}

// G2 = false: eight math warps process the two 64-query halves of a step one after the other (320 threads).
// G2 = true: sixteen math warps in two groups of eight, group h owning half h of every step and dQ columns [32 h, 32 h + 32)
// (576 threads, at most 112 registers each: a warp's 32 columns are read in two passes of 16).  The elementwise phase is bound by
// latency (TMEM loads, special-function unit, barriers), not by issue slots, so twice the warps nearly halve it.
template <bool G2>
__global__ void __launch_bounds__(G2 ? 576 : 320, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapdO,
                const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                const __grid_constant__ CUtensorMap mapK2, const __grid_constant__ CUtensorMap mapV2,
                const __grid_constant__ CUtensorMap mapdQ, const AttnBwdParams p) {
  using L = BwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + L::TILE;
  uint8_t* sST = sV + L::TILE;                               // stages: [Q tile | dO tile]
  uint8_t* sDS = sST + L::STAGES * 2 * L::TILE;              // two dS^T tiles (steps alternate)
  float* sDQ = reinterpret_cast<float*>(sDS + 2 * L::DS_BYTES);    // [128 queries][64] f32, the step's dQ tile
  float* sLSE = sDQ + 128 * HD;                              // [2][128], premultiplied by log2(e)
  float* sDel = sLSE + 2 * 128;                              // [2][128], premultiplied by scale
  int* sE1 = reinterpret_cast<int*>(sDel + 2 * 128);         // [2][128] per query column: last key of the prefix interval
  int* sS2 = sE1 + 2 * 128;                                  // [2][128] second interval
  int* sE2 = sS2 + 2 * 128;
  int4* items = reinterpret_cast<int4*>(sE2 + 2 * 128);      // see build_work_items
  uint64_t* bars = reinterpret_cast<uint64_t*>(items + MAX_ITEMS);
  // everything carved above plus the barrier block must fit what the launcher asks for (1024 bytes of alignment slack included)
  static_assert(2 * L::TILE + L::STAGES * 2 * L::TILE + 2 * L::DS_BYTES + L::DQ_BYTES + L::AUX + L::MASK + L::ITEMS + 256 + 1024 <= L::TOTAL,
                "shared-memory layout exceeds BwdSmem::TOTAL");
  static_assert(L::TOTAL <= 227 * 1024, "shared memory per CTA");
  uint64_t* kv_full = bars;
  uint64_t* st_full = bars + 1;                              // [2]
  uint64_t* st_empty = st_full + 2;                          // [2]
  uint64_t* s_full = st_empty + 2;                           // [2] one per 64-query half
  uint64_t* pds_ready = s_full + 2;                          // [2]
  uint64_t* dq_full = pds_ready + 2;
  uint64_t* dq_empty = dq_full + 1;
  uint64_t* acc_final = dq_empty + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_final + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* n_items_slot = const_cast<int*>(abort_word) + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int jb = blockIdx.x, hk = blockIdx.y, b = blockIdx.z;
  const int rep = p.nh / p.nkv;
  // ---- which key block this CTA owns, and the work items that see it (one thread; a few hundred cheap tests at most)
  const OwnedBlock own = owned_block(p, jb, b);
  if (!own.live) return;
  const bool second = own.second;
  const int kseq = own.kseq, krow = own.krow, klen = own.klen;
  if (threadIdx.x == 0) *n_items_slot = build_work_items(p, own, jb, b, items);
  // (published by the __syncthreads below)
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t C_S = 0, C_DP = 128, C_DV = 256, C_DK = 320, C_DQ = 384;
  constexpr int NMATH = G2 ? 512 : 256;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&st_full[s], 1); mbar_init(&st_empty[s], 1);
      mbar_init(&s_full[s], 1); mbar_init(&pds_ready[s], 256);
    }
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, NMATH);
    mbar_init(acc_final, 1);
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapdO); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV); tma_prefetch_desc(&mapK2); tma_prefetch_desc(&mapV2); tma_prefetch_desc(&mapdQ);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  int nq_it = *n_items_slot;
  if (nq_it > MAX_ITEMS) {                                   // the launcher sizes the list; never expected
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ERR_WORK_LIST);
    nq_it = 0;
  }
  const int n_it = rep * nq_it;                              // heads of the group outermost, work items inside

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one() && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * L::TILE);
      tma_load_4d_b(sK, second ? &mapK2 : &mapK, kv_full, 0, hk, krow, kseq);
      tma_load_4d_b(sV, second ? &mapV2 : &mapV, kv_full, 0, hk, krow, kseq);
      int ii = 0, h = hk * rep;                              // item index and head of step `it`
      for (int it = 0; it < n_it; ++it) {
        const int s = it & 1;
        if (!mbar_wait_bounded(&st_empty[s], ((it >> 1) & 1) ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) break;
        const int4 item = items[ii];
        const int qt = item_qt(item);
        uint8_t* sQ = sST + s * 2 * L::TILE;
        mbar_expect_tx(&st_full[s], 2 * L::TILE);
        tma_load_4d_b(sQ, &mapQ, &st_full[s], 0, h, qt * BQ, item.x);
        tma_load_4d_b(sQ + L::TILE, &mapdO, &st_full[s], 0, h, qt * BQ, item.x);
        if (++ii == nq_it) { ii = 0; ++h; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one() && n_it > 0) {
      const uint32_t id_s = make_idesc_bf16(128, 64, 0, 0);         // S^T, dP^T of one 64-query half: operands K-major
      const uint32_t id_kv = make_idesc_bf16(128, HD, 0, 1);        // dV, dK: A from TMEM, B = [q rows, d] N-major
      const uint32_t id_q = make_idesc_bf16(128, HD, 1, 1);         // dQ: A = dS^T (M-major), B = K (N-major)
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_word, p.status, ERR_WAIT_FULL);
      // S^T and dP^T of half `hf` of step `it` (its Q / dO stage must be full)
      auto issue_scores = [&](int it, int hf) {
        const uint32_t aQ = smem_u32(sST + (it & 1) * 2 * L::TILE), aDO = aQ + L::TILE;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem + C_S + hf * 64, make_smem_desc(aK + k * 32, 16, 1024), make_smem_desc(aQ + hf * 8192 + k * 32, 16, 1024), id_s, k ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < HD / 16; ++k)
          umma_f16(tmem + C_DP + hf * 64, make_smem_desc(aV + k * 32, 16, 1024), make_smem_desc(aDO + hf * 8192 + k * 32, 16, 1024), id_s, k ? 1u : 0u);
        umma_commit(&s_full[hf]);
      };
      // dV += P^T dO and dK += dS^T Q over the 64 queries of half `hf`
      auto issue_kv = [&](int it, int hf) {
        const uint32_t aQ = smem_u32(sST + (it & 1) * 2 * L::TILE), aDO = aQ + L::TILE;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ts(tmem + C_DV, tmem + C_S + hf * 64 + k * 8, make_smem_desc(aDO + hf * 8192 + k * 2048, 16384, 1024), id_kv,
                      (it | hf | k) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ts(tmem + C_DK, tmem + C_DP + hf * 64 + k * 8, make_smem_desc(aQ + hf * 8192 + k * 2048, 16384, 1024), id_kv,
                      (it | hf | k) ? 1u : 0u);
      };
      if (ok) ok = mbar_wait_bounded(&st_full[0], 0, abort_word, p.status, ERR_WAIT_FULL);
      if (ok) { tc_fence_after(); issue_scores(0, 0); issue_scores(0, 1); }
      for (int it = 0; it < n_it && ok; ++it) {
        const bool more = it + 1 < n_it;
        if (!mbar_wait_bounded(&pds_ready[0], it & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_kv(it, 0);
        if (more) {
          if (!mbar_wait_bounded(&st_full[(it + 1) & 1], ((it + 1) >> 1) & 1, abort_word, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          issue_scores(it + 1, 0);                                   // half 0's columns are free once dV / dK above have run
        }
        if (!mbar_wait_bounded(&pds_ready[1], it & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_kv(it, 1);
        umma_commit(&st_empty[it & 1]);                               // Q and dO of this step are consumed
        if (!mbar_wait_bounded(dq_empty, (it & 1) ^ 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t aDS = smem_u32(sDS + (it & 1) * L::DS_BYTES);
#pragma unroll
        for (int k = 0; k < BKEY / 16; ++k)                          // contraction over the 128 keys of the block
          umma_f16(tmem + C_DQ, make_smem_desc(aDS + k * 2048, 16384, 1024), make_smem_desc(aK + k * 2048, 16384, 1024), id_q, k ? 1u : 0u);
        umma_commit(dq_full);
        if (more) issue_scores(it + 1, 1);
      }
      if (ok) umma_commit(acc_final);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax backward, dQ reduction, dK / dV stores
    const int w = warp - 2;                                  // 0..7 (or 0..15)
    const int quarter = warp & 3;                            // TMEM lane quarter of this warp
    const int sub = (w >> 2) & 1;                            // which 32 of a half's 64 query columns
    const int grp = G2 ? (w >> 3) : 0;                       // G2: the 64-query half (and dQ column half) this warp works on
    const int gt = (threadIdx.x - 64) & 255;                 // thread within its group of eight warps
    const int kr = quarter * 32 + lane;                      // key row within the block == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const int bar_a = 1 + 3 * grp, bar_b = 2 + 3 * grp, bar_c = 3 + 3 * grp;     // named barriers of this group (256 threads)
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr float LOG2E = 1.4426950408889634f;
    bool ok = n_it > 0;
    // LSE, D and (for tiles that need the mask) the visible key intervals of the step's queries.  G1: thread t < 128 serves query
    // t (LSE, intervals), thread 128 + t its D.  G2: group h serves queries 64 h ... 64 h + 63 the same way with 64 + 64 threads.
    constexpr int NQ = G2 ? 64 : 128;                        // queries a group serves
    const int q_loc = grp * 64 + (gt & (NQ - 1));            // query row within the tile this thread serves (gt < 2 NQ)
    auto load_aux = [&](const int4& item, int h, float& val, int& e1, int& s2, int& e2) {
      const int qi = item_qt(item) * BQ + q_loc;
      const long long base = ((long long)item.x * p.nh + h) * p.Cq;
      if (gt < NQ) {
        val = (qi < p.Cq) ? p.lse[base + qi] * LOG2E : 1e30f;
        if (item.y & 1) {                                    // positions RELATIVE to this block's first row
          const RowMask rm = item_row_mask(p, item, qi);
          e1 = rm.e1; s2 = rm.s2; e2 = rm.e2;
        }
      } else if (gt < 2 * NQ) {
        val = (qi < p.Cq) ? p.delta[base + qi] * p.scale : 0.f;
      }
    };
    auto store_aux = [&](int buf, float val, int e1, int s2, int e2) {
      const int x = buf * 128 + q_loc;
      if (gt < NQ) { sLSE[x] = val; sE1[x] = e1; sS2[x] = s2; sE2[x] = e2; } else if (gt < 2 * NQ) sDel[x] = val;
    };
    // add the dQ tile of a step (lanes = queries) into global memory: the warps copy it from TMEM into shared memory (two
    // [128 x 32] f32 boxes, rows of 128 bytes with the 16-byte pieces XOR-swizzled by row: the tensor map's 128-byte swizzle,
    // which also spreads the lanes' stores over the banks) and one thread per box issues a bulk tensor reduction (f32 add);
    // rows past the end of the sequence are clipped by the tensor map.  G2: each group owns one box.
    auto reduce_dq = [&](int it, const int4& item, int h) -> bool {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(dq_full, it & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (gt == 0) bulk_wait_read0();                        // the previous reduction has finished reading the tile
      if (!bar_red_and(bar_c, 256, got)) return false;
      tc_fence_after();
      const int qt = item_qt(item);
      if constexpr (!G2) {
        uint32_t r[32];
        tmem_ld_32x32(tmem + C_DQ + lane_addr + sub * 32, r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(dq_empty);
        float* row = sDQ + sub * (128 * 32) + kr * 32;        // the lane index doubles as the query row here
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<float4*>(row + 4 * (j ^ (kr & 7))) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                               __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        fence_async_proxy();
        bar_sync_named(bar_b, 256);
        if (gt == 0) {
          tma_reduce_add_4d(&mapdQ, sDQ, 0, h, qt * BQ, item.x);
          tma_reduce_add_4d(&mapdQ, sDQ + 128 * 32, 32, h, qt * BQ, item.x);
          bulk_commit();
        }
      } else {
        uint32_t r[16];
        tmem_ld_32x16(tmem + C_DQ + lane_addr + grp * 32 + sub * 16, r);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(dq_empty);
        float* row = sDQ + grp * (128 * 32) + kr * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          *reinterpret_cast<float4*>(row + 4 * ((sub * 4 + j) ^ (kr & 7))) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                                           __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        fence_async_proxy();
        bar_sync_named(bar_b, 256);
        if (gt == 0) {
          tma_reduce_add_4d(&mapdQ, sDQ + grp * (128 * 32), grp * 32, h, qt * BQ, item.x);
          bulk_commit();
        }
      }
      return true;
    };
    // P^T and dS^T (bf16 pairs) of W query columns starting at tile column c0, from the raw S^T / dP^T columns
    auto softmax_bwd_cols = [&](auto& sr, auto& dr, int c0, int width, uint32_t* pp, uint32_t* dd, const float* lse2, const float* del,
                                const int* e1s, const int* s2s, const int* e2s, bool need_mask) {
#pragma unroll
      for (int i = 0; i < width; i += 4) {
        const float4 l4 = *reinterpret_cast<const float4*>(lse2 + c0 + i);     // broadcast reads
        const float4 d4 = *reinterpret_cast<const float4*>(del + c0 + i);      // D * scale
        const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
        float pv[4], dv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          float pe = ex2_approx(fmaf(__uint_as_float(sr[i + u]), sl2, -lv[u]));
          if (need_mask) {
            const int q = c0 + i + u;                        // query column; visible: kr <= e1 or s2 <= kr <= e2 (block-relative)
            if (kr > e1s[q] && (kr < s2s[q] || kr > e2s[q])) pe = 0.f;
          }
          pv[u] = pe;
          dv[u] = pe * fmaf(__uint_as_float(dr[i + u]), p.scale, -dl[u]);
        }
#pragma unroll
        for (int u = 0; u < 4; u += 2) {
          __nv_bfloat162 pb = __floats2bfloat162_rn(pv[u], pv[u + 1]);
          __nv_bfloat162 db = __floats2bfloat162_rn(dv[u], dv[u + 1]);
          pp[(i + u) / 2] = *reinterpret_cast<uint32_t*>(&pb);
          dd[(i + u) / 2] = *reinterpret_cast<uint32_t*>(&db);
        }
      }
    };
    int ii = 0, h = hk * rep;                                // item index and head of step `it`
    int4 item = make_int4(0, 0, 0, 0), prev_item = item;
    int prev_h = h;
    if (ok) {
      item = items[0];
      float v0 = 0.f;
      int a0 = 0, a1 = 0, a2 = 0;
      load_aux(item, h, v0, a0, a1, a2);
      store_aux(0, v0, a0, a1, a2);
    }
    for (int it = 0; it < n_it && ok; ++it) {
      // the next step's item and head (counters, not divisions), and its LSE / D / intervals on their way
      int ii_n = ii + 1, h_n = h;
      if (ii_n == nq_it) { ii_n = 0; ++h_n; }
      float vnext = 0.f;
      int n1 = 0, n2 = 0, n3 = 0;
      int4 next_item = item;
      if (it + 1 < n_it) { next_item = items[ii_n]; load_aux(next_item, h_n, vnext, n1, n2, n3); }
      const float* lse2 = sLSE + (it & 1) * 128;
      const float* del = sDel + (it & 1) * 128;
      const int* e1s = sE1 + (it & 1) * 128;
      const int* s2s = sS2 + (it & 1) * 128;
      const int* e2s = sE2 + (it & 1) * 128;
      const bool need_mask = (item.y & 1) != 0;
      uint8_t* ds_tile = sDS + (it & 1) * L::DS_BYTES;
#pragma unroll 1
      for (int hf = grp; hf < (G2 ? grp + 1 : 2) && ok; ++hf) {
        int got = 1;
        if (lane == 0) got = mbar_wait_bounded(&s_full[hf], it & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        // one verdict for the group's eight warps (they meet at barriers below); it also publishes this step's LSE / D
        if (!bar_red_and(bar_a, 256, got)) { ok = false; break; }
        tc_fence_after();
        const int c0 = hf * 64 + sub * 32;                   // first query column of this warp in this half
        uint32_t pp[16], dd[16];
        if constexpr (!G2) {
          uint32_t sr[32], dr[32];
          tmem_ld_32x32(tmem + C_S + lane_addr + c0, sr);
          tmem_ld_32x32(tmem + C_DP + lane_addr + c0, dr);
          tmem_ld_wait();
          softmax_bwd_cols(sr, dr, c0, 32, pp, dd, lse2, del, e1s, s2s, e2s, need_mask);
        } else {
#pragma unroll
          for (int ps = 0; ps < 2; ++ps) {
            uint32_t sr[16], dr[16];
            tmem_ld_32x16(tmem + C_S + lane_addr + c0 + ps * 16, sr);
            tmem_ld_32x16(tmem + C_DP + lane_addr + c0 + ps * 16, dr);
            tmem_ld_wait();
            softmax_bwd_cols(sr, dr, c0 + ps * 16, 16, pp + ps * 8, dd + ps * 8, lse2, del, e1s, s2s, e2s, need_mask);
          }
        }
        // every warp that reads this half's columns has read them: the packed results may now overwrite them
        tc_fence_before();
        bar_sync_named(bar_b, 256);
        tc_fence_after();
        tmem_st_32x16(tmem + C_S + lane_addr + hf * 64 + sub * 16, pp);     // 32 queries -> 16 columns of bf16 pairs
        tmem_st_32x16(tmem + C_DP + lane_addr + hf * 64 + sub * 16, dd);
        {
          // dS^T row kr, queries c0..c0+31, into the M-major A tile: 64-query block hf, 128-byte rows indexed by key
          uint8_t* base = ds_tile + hf * (128 * 128) + (kr / 8) * 1024 + (kr % 8) * 128;
#pragma unroll
          for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4*>(base + (((sub * 4 + q) ^ (kr % 8)) * 16)) = make_uint4(dd[4 * q], dd[4 * q + 1], dd[4 * q + 2], dd[4 * q + 3]);
        }
        tmem_st_wait();
        fence_async_proxy();
        tc_fence_before();
        mbar_arrive(&pds_ready[hf]);
        // the previous step's dQ, while the tensor core works on this step's products
        if ((G2 || hf == 0) && it > 0) ok = reduce_dq(it - 1, prev_item, prev_h);
      }
      if (!ok) break;
      // next step's LSE / D into the other buffer (its last readers passed this group's first barrier of this step)
      if (it + 1 < n_it) store_aux((it + 1) & 1, vnext, n1, n2, n3);
      prev_item = item; prev_h = h;
      item = next_item; ii = ii_n; h = h_n;
    }
    if (ok) ok = reduce_dq(n_it - 1, prev_item, prev_h);
    if (gt == 0) bulk_wait0();                               // the last dQ reduction has been performed
    // dK, dV of the block: a warp's 32 (G2: 16) of the 64 columns
    constexpr int CW = G2 ? 16 : 32;
    const int col = G2 ? grp * 32 + sub * 16 : sub * 32;
    if (ok) {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(acc_final, 0, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got) {
        tc_fence_after();
        uint32_t rv[CW], rk[CW];
        if constexpr (G2) {
          tmem_ld_32x16(tmem + C_DV + lane_addr + col, rv);
          tmem_ld_32x16(tmem + C_DK + lane_addr + col, rk);
        } else {
          tmem_ld_32x32(tmem + C_DV + lane_addr + col, rv);
          tmem_ld_32x32(tmem + C_DK + lane_addr + col, rk);
        }
        tmem_ld_wait();
        if (krow + kr < klen) {
          __nv_bfloat16* outK = second ? p.dK2 : p.dK;
          __nv_bfloat16* outV = second ? p.dV2 : p.dV;
          const long long o = (((long long)kseq * klen + krow + kr) * p.nkv + hk) * HD + col;
#pragma unroll
          for (int i = 0; i < CW; i += 8) {
            uint4 v, k;
            __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
            __nv_bfloat162* kb = reinterpret_cast<__nv_bfloat162*>(&k);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              vb[q] = __floats2bfloat162_rn(__uint_as_float(rv[i + 2 * q]), __uint_as_float(rv[i + 2 * q + 1]));
              kb[q] = __floats2bfloat162_rn(__uint_as_float(rk[i + 2 * q]), __uint_as_float(rk[i + 2 * q + 1]));
            }
            *reinterpret_cast<uint4*>(outV + o + i) = v;
            *reinterpret_cast<uint4*>(outK + o + i) = k;
          }
        }
      }
    } else if (n_it == 0 && krow + kr < klen) {
      // no query sees this key block: its gradients are zero
      const long long o = (((long long)kseq * klen + krow + kr) * p.nkv + hk) * HD + col;
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < CW; i += 8) {
        *reinterpret_cast<uint4*>((second ? p.dV2 : p.dV) + o + i) = z;
        *reinterpret_cast<uint4*>((second ? p.dK2 : p.dK) + o + i) = z;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

typedef CUresult (*EncodeTiledFnB)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnB bwd_encode_fn() {
  static EncodeTiledFnB fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFnB>(ptr);
  });
  return fn;
}

// f32 [n, rows, heads, hd], box = 32 x 1 head x 128 rows x 1, 128-byte swizzle: the dQ accumulation target of the bulk reduction
static int make_map4f(CUtensorMap* map, const void* ptr, int n, int rows, int heads, int hd) {
  EncodeTiledFnB enc = bwd_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)hd * 4, (cuuint64_t)heads * hd * 4, (cuuint64_t)rows * heads * hd * 4};
  cuuint32_t box[4] = {32, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (int c = check_map(ptr, 4, dims, strides, 4)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

static int make_map4b(CUtensorMap* map, const void* ptr, int n, int rows, int heads, int hd, long long batch_stride = 0) {
  EncodeTiledFnB enc = bwd_encode_fn();
  if (!enc) return -1;
  if (batch_stride <= 0) batch_stride = (long long)rows * heads * hd;
  cuuint64_t dims[4] = {(cuuint64_t)hd, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)hd * 2, (cuuint64_t)heads * hd * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (int c = check_map(ptr, 4, dims, strides, 2)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace dttt

using namespace dttt;

namespace dttt {
// the head-dimension-128 kernel (attn_bwd128_tcgen05.cu): same maps with 128-wide rows, same parameter block
int attn_bwd128_launch(dim3 grid, const CUtensorMap& mq, const CUtensorMap& mdo, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mk2, const CUtensorMap& mv2, const CUtensorMap& mdq, const AttnBwdParams& p, const void* O,
                       const void* dO, float* delta, long long q_rows, cudaStream_t stream);

static int launch_bwd(dim3 grid, const CUtensorMap& mq, const CUtensorMap& mdo, const CUtensorMap& mk, const CUtensorMap& mv,
                      const CUtensorMap& mk2, const CUtensorMap& mv2, const CUtensorMap& mdq, const AttnBwdParams& p,
                      const void* O, const void* dO, float* delta, long long q_rows, int d, cudaStream_t stream) {
  if (d == 128) return attn_bwd128_launch(grid, mq, mdo, mk, mv, mk2, mv2, mdq, p, O, dO, delta, q_rows, stream);
  attn_bwd_delta_kernel<<<(unsigned)((q_rows * 8 + 255) / 256), 256, 0, stream>>>(
      reinterpret_cast<const __nv_bfloat16*>(O), reinterpret_cast<const __nv_bfloat16*>(dO), delta, q_rows, p.Cq, p.nh);
  // sixteen math warps unless DTTT_ATTN_BWD_WARPS=8 asks for the eight-warp form
  static const bool sixteen = [] { const char* e = getenv("DTTT_ATTN_BWD_WARPS"); return !(e && e[0] == '8'); }();
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(attn_bwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL);
    cudaFuncSetAttribute(attn_bwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, BwdSmem::TOTAL);
    attr = true;
  }
  if (sixteen) attn_bwd_kernel<true><<<grid, 576, BwdSmem::TOTAL, stream>>>(mq, mdo, mk, mv, mk2, mv2, mdq, p);
  else attn_bwd_kernel<false><<<grid, 320, BwdSmem::TOTAL, stream>>>(mq, mdo, mk, mv, mk2, mv2, mdq, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
}  // namespace dttt

// Every last dimension below is the head dimension d, 64 or 128.  Q, O, dO [n, Cq, nh, 64] (bf16, contiguous); keys / values as one or two pairs like dttt_attn_fwd (K2 == null: one pair):
// K / V [n, Kn1, nkv, 64] with `k_bs` / `v_bs` elements between sequences, K2 / V2 [n, Kn2, nkv, 64]; dK / dV [n, Kn1, nkv, 64]
// and dK2 / dV2 [n, Kn2, nkv, 64] contiguous outputs; lse [n, nh, Cq] f32 from the forward; delta [n, nh, Cq] f32 scratch
// (written here); dQ [n, Cq, nh, 64] f32, must be zero on entry (accumulated into).  mode / param: the own-chunk pattern as in
// dttt_attn_fwd_masked (Cq a multiple of 128 for modes 2-4).
extern "C" int dttt_attn_bwd_masked(const void* Q, const void* K, const void* V, const void* K2, const void* V2, const void* O,
                                    const void* dO, const float* lse, float* delta, float* dQ, void* dK, void* dV, void* dK2, void* dV2,
                                    int n, int Cq, int Kn1, int Kn2, int nh, int nkv, int d, long long k_bs, long long v_bs,
                                    long long k2_bs, long long v2_bs, float scale, int mode, int param, int* status,
                                    cudaStream_t stream) {
  const int Kn = Kn1 + (K2 ? Kn2 : 0);
  if ((d != 64 && d != 128) || nh % nkv || n <= 0 || Cq <= 0 || Kn < Cq || mode < 0 || mode > MASK_READ) return -2;
  if (mode >= MASK_SPLIT && (Cq % BKEY || param <= 0 || param > Cq)) return -3;
  if (mode == MASK_READ && Kn < 2 * Cq) return -3;
  if (K2 && Kn1 % BKEY) return -4;
  if ((Cq + BQ - 1) / BQ > MAX_ITEMS) return -5;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { int dev = 0; cudaGetDevice(&dev); cudaSetDevice(dev); cudaFree(0); ctx_bound = true; }
  CUtensorMap mq, mdo, mk, mv, mk2, mv2, mdq;
  int r;
  if ((r = make_map4f(&mdq, dQ, n, Cq, nh, d))) return 500 + r;
  if ((r = make_map4b(&mq, Q, n, Cq, nh, d))) return 100 + r;
  if ((r = make_map4b(&mdo, dO, n, Cq, nh, d))) return 200 + r;
  if (Kn1 > 0) {
    if ((r = make_map4b(&mk, K, n, Kn1, nkv, d, k_bs))) return 300 + r;
    if ((r = make_map4b(&mv, V, n, Kn1, nkv, d, v_bs))) return 400 + r;
  }
  if (K2) {
    if ((r = make_map4b(&mk2, K2, n, Kn2, nkv, d, k2_bs))) return 600 + r;
    if ((r = make_map4b(&mv2, V2, n, Kn2, nkv, d, v2_bs))) return 700 + r;
    if (Kn1 == 0) { mk = mk2; mv = mv2; }
  } else {
    mk2 = mk; mv2 = mv;
  }
  AttnBwdParams p;
  memset(&p, 0, sizeof(p));
  p.n = n; p.Cq = Cq; p.Kn = Kn; p.Kn1 = K2 ? Kn1 : Kn; p.nh = nh; p.nkv = nkv; p.causal = mode == MASK_CAUSAL; p.scale = scale;
  p.mask_mode = mode; p.mask_param = param;
  p.lse = lse; p.delta = delta; p.dQ = dQ;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dK); p.dV = reinterpret_cast<__nv_bfloat16*>(dV);
  p.dK2 = reinterpret_cast<__nv_bfloat16*>(dK2); p.dV2 = reinterpret_cast<__nv_bfloat16*>(dV2); p.status = status;
  dim3 grid((Kn + BKEY - 1) / BKEY, nkv, n);
  return launch_bwd(grid, mq, mdo, mk, mv, mk2, mv2, mdq, p, O, dO, delta, (long long)n * Cq * nh, d, stream);
}

extern "C" int dttt_attn_bwd(const void* Q, const void* K, const void* V, const void* K2, const void* V2, const void* O, const void* dO,
                             const float* lse, float* delta, float* dQ, void* dK, void* dV, void* dK2, void* dV2, int n, int Cq,
                             int Kn1, int Kn2, int nh, int nkv, int d, long long k_bs, long long v_bs, long long k2_bs,
                             long long v2_bs, float scale, int causal, int* status, cudaStream_t stream) {
  return dttt_attn_bwd_masked(Q, K, V, K2, V2, O, dO, lse, delta, dQ, dK, dV, dK2, dV2, n, Cq, Kn1, Kn2, nh, nkv, d, k_bs, v_bs, k2_bs,
                              v2_bs, scale, causal ? MASK_CAUSAL : MASK_FULL, 0, status, stream);
}

// Backward of dttt_attn_fwd_segment.  Q, O, dO [B, streams, chunks * C, nh, 64]; Kc / Vc the clean buffer [B, (W + chunks) C, nkv, 64]
// (`kc_bs` / `vc_bs` elements between sequences); Ko / Vo [B, streams, chunks * C, nkv, 64]; lse, delta [B * streams * chunks, nh, C];
// dQ f32 like Q, zero on entry.  Outputs: dKc / dVc [B, (W + chunks) C, nkv, 64] contiguous (the gradient of every clean key from
// every chunk that had it in its window AND from the clean stream's own chunk, summed on chip); dKo / dVo [B, streams, chunks * C,
// nkv, 64] for the other streams' own keys (the clean stream's slot is not written: its own keys are rows of the clean buffer).
// The clean stream is stream 1.
extern "C" int dttt_attn_bwd_segment(const void* Q, const void* Kc, const void* Vc, const void* Ko, const void* Vo, const void* O,
                                     const void* dO, const float* lse, float* delta, float* dQ, void* dKc, void* dVc, void* dKo, void* dVo,
                                     int B, int streams, int chunks, int C, int W, int first, int reach, int nh, int nkv, int d,
                                     long long kc_bs, long long vc_bs, const int* modes, const int* params, float scale, int* status,
                                     cudaStream_t stream) {
  if ((d != 64 && d != 128) || nh % nkv || B <= 0 || streams < 2 || streams > MAX_STREAMS || chunks <= 0 || C % BKEY || W < 0) return -2;
  if (streams * (W + 1) * (C / BQ) > MAX_ITEMS) return -5;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { int dev = 0; cudaGetDevice(&dev); cudaSetDevice(dev); cudaFree(0); ctx_bound = true; }
  const int n = B * streams * chunks;
  CUtensorMap mq, mdo, mk, mv, mk2, mv2, mdq;
  int r;
  if ((r = make_map4f(&mdq, dQ, n, C, nh, d))) return 500 + r;
  if ((r = make_map4b(&mq, Q, n, C, nh, d))) return 100 + r;
  if ((r = make_map4b(&mdo, dO, n, C, nh, d))) return 200 + r;
  if ((r = make_map4b(&mk, Kc, B, (W + chunks) * C, nkv, d, kc_bs))) return 300 + r;
  if ((r = make_map4b(&mv, Vc, B, (W + chunks) * C, nkv, d, vc_bs))) return 400 + r;
  if ((r = make_map4b(&mk2, Ko, B * streams, chunks * C, nkv, d))) return 600 + r;
  if ((r = make_map4b(&mv2, Vo, B * streams, chunks * C, nkv, d))) return 700 + r;
  AttnBwdParams p;
  memset(&p, 0, sizeof(p));
  p.n = n; p.Cq = C; p.nh = nh; p.nkv = nkv; p.scale = scale;
  p.sg.on = 1; p.sg.streams = streams; p.sg.chunks = chunks; p.sg.first = first; p.sg.W = W; p.sg.reach = reach;
  for (int s = 0; s < streams; ++s) {
    if (modes[s] < 0 || modes[s] >= MASK_READ || (modes[s] >= MASK_SPLIT && (params[s] <= 0 || params[s] > C))) return -3;
    p.sg.mode[s] = modes[s]; p.sg.param[s] = params[s];
  }
  p.lse = lse; p.delta = delta; p.dQ = dQ;
  p.dK = reinterpret_cast<__nv_bfloat16*>(dKc); p.dV = reinterpret_cast<__nv_bfloat16*>(dVc);
  p.dK2 = reinterpret_cast<__nv_bfloat16*>(dKo); p.dV2 = reinterpret_cast<__nv_bfloat16*>(dVo); p.status = status;
  dim3 grid((W + chunks) * C / BKEY, nkv, B * streams);
  return launch_bwd(grid, mq, mdo, mk, mv, mk2, mv2, mdq, p, O, dO, delta, (long long)n * C * nh, d, stream);
}
