// Chunk-window flash attention, backward, head dimension 128 (the reference model's own geometry: 16 / 4 heads of 128).
//
// Same algorithm, work lists and masks as attn_bwd_tcgen05.cu (head dimension 64): one CTA owns a block of 128 keys, walks
// the (sequence, query tile) work items that see it for every query head of the group, keeps dV and dK of the block in tensor
// memory over the whole walk, and adds each step's dQ tile into an f32 buffer by bulk tensor reductions.
//
// What changes with 128-wide heads is the budget.  Tensor memory: dV, dK and dQ take 128 columns each, which leaves 128 of the
// 512 for the scores, so a step's two 64-query halves SHARE one S^T (64 columns) and one dP^T (64 columns) instead of having
// their own: the issuer runs scores(half 0), dV / dK(half 0), scores(half 1), dV / dK(half 1), dQ in that order and the in-order
// tensor pipe makes the reuse safe.  Shared memory: K, V, Q and dO tiles are 32 KB each, so Q / dO have one stage and dS^T
// one buffer (the dQ product of a step is issued before the next step's scores, so nothing overwrites what it still reads),
// and the f32 dQ tile is staged 64 columns at a time.
//
//   warp 0      TMA: K, V once; Q and dO of every step
//   warp 1      tcgen05.mma issuer, TMEM owner
//   warps 2-9   two per TMEM lane quarter: softmax-backward math, dQ reduction, final dK / dV stores
// TMEM columns: S^T / P^T [0,64)  dP^T / dS^T [64,128)  dV [128,256)  dK [256,384)  dQ [384,512).
// Every wait is bounded (ptx_sm100.cuh); on a timeout the roles leave through the common exit and TMEM is freed.
#include "attn_bwd_common.cuh"

#include <cstdlib>

namespace dttt {
namespace b128 {

constexpr int HD = 128;
constexpr int SUB = 128 * 128;                    // bytes of one [128 rows x 64 d] sub-tile (128-byte swizzled rows)

struct Smem {
  static constexpr int TILE = 2 * SUB;                       // one [128, 128] bf16 tile: two d sub-tiles
  static constexpr int DS_BYTES = 128 * 128 * 2;
  static constexpr int DQ_BYTES = 128 * 64 * 4;              // 64 columns of the dQ tile at a time
  static constexpr int AUX = 2 * 2 * 128 * 4;
  static constexpr int MASK = 2 * 3 * 128 * 4;
  static constexpr int ITEMS = MAX_ITEMS * 16;
  static constexpr int TOTAL = 4 * TILE + DS_BYTES + DQ_BYTES + AUX + MASK + ITEMS + 1024 + 1024;
};

// delta[b, h, i] = sum_d dO[b, i, h, d] * O[b, i, h, d]; sixteen threads per row of 128.
__global__ void delta_kernel(const __nv_bfloat16* __restrict__ O, const __nv_bfloat16* __restrict__ dO, float* __restrict__ delta,
                             long long rows, int Cq, int nh) {
  const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = gid >> 4;
  const int part = (int)(gid & 15);
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
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (part == 0 && row < rows) {
    const long long bi = row / nh;
    const int h = (int)(row - bi * nh);
    const long long b = bi / Cq;
    const int i = (int)(bi - b * Cq);
    delta[(b * nh + h) * Cq + i] = acc;
  }
}

// W16 = false: eight math warps, 32 query columns of a half per thread.  W16 = true: sixteen math warps, 16 columns per thread
// (576 threads, at most 96 registers): the halves of a step cannot overlap here (they share their score columns), so the
// elementwise phase is on the critical path and twice the warps shorten it.
template <bool W16>
__global__ void __launch_bounds__(W16 ? 576 : 320, 1)
attn_bwd128_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapdO,
                   const __grid_constant__ CUtensorMap mapK, const __grid_constant__ CUtensorMap mapV,
                   const __grid_constant__ CUtensorMap mapK2, const __grid_constant__ CUtensorMap mapV2,
                   const __grid_constant__ CUtensorMap mapdQ, const AttnBwdParams p) {
  using L = Smem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + L::TILE;
  uint8_t* sQ = sV + L::TILE;                                // the step's Q tile, then its dO tile
  uint8_t* sDO = sQ + L::TILE;
  uint8_t* sDS = sDO + L::TILE;                              // dS^T for the dQ product
  float* sDQ = reinterpret_cast<float*>(sDS + L::DS_BYTES);  // [2 boxes][128 queries][32] f32
  float* sLSE = sDQ + 128 * 64;                              // [2][128], premultiplied by log2(e)
  float* sDel = sLSE + 2 * 128;                              // [2][128], premultiplied by scale
  int* sE1 = reinterpret_cast<int*>(sDel + 2 * 128);
  int* sS2 = sE1 + 2 * 128;
  int* sE2 = sS2 + 2 * 128;
  int4* items = reinterpret_cast<int4*>(sE2 + 2 * 128);      // see build_work_items
  uint64_t* bars = reinterpret_cast<uint64_t*>(items + MAX_ITEMS);
  static_assert(4 * L::TILE + L::DS_BYTES + L::DQ_BYTES + L::AUX + L::MASK + L::ITEMS + 256 + 1024 <= L::TOTAL, "shared-memory layout");
  static_assert(L::TOTAL <= 227 * 1024, "shared memory per CTA");
  uint64_t* kv_full = bars;
  uint64_t* st_full = bars + 1;
  uint64_t* st_empty = bars + 2;
  uint64_t* s_full = bars + 3;                               // [2] one per 64-query half
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
  const OwnedBlock own = owned_block(p, jb, b);
  if (!own.live) return;
  const bool second = own.second;
  const int kseq = own.kseq, krow = own.krow, klen = own.klen;
  if (threadIdx.x == 0) *n_items_slot = build_work_items(p, own, jb, b, items);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t C_S = 0, C_DP = 64, C_DV = 128, C_DK = 256, C_DQ = 384;
  constexpr int NM = W16 ? 512 : 256;                        // math threads
  constexpr int CW = W16 ? 16 : 32;                          // query columns of a half per thread

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(st_full, 1); mbar_init(st_empty, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&pds_ready[s], NM); }
    mbar_init(dq_full, 1);
    mbar_init(dq_empty, NM);
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
  if (nq_it > MAX_ITEMS) {
    if (threadIdx.x == 0) atomicCAS(p.status, 0, ERR_WORK_LIST);
    nq_it = 0;
  }
  const int n_it = rep * nq_it;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one() && n_it > 0) {
      mbar_expect_tx(kv_full, 2 * L::TILE);
#pragma unroll
      for (int db = 0; db < 2; ++db) {
        tma_load_4d_b(sK + db * SUB, second ? &mapK2 : &mapK, kv_full, db * 64, hk, krow, kseq);
        tma_load_4d_b(sV + db * SUB, second ? &mapV2 : &mapV, kv_full, db * 64, hk, krow, kseq);
      }
      int ii = 0, h = hk * rep;                              // item index and head of step `it`
      for (int it = 0; it < n_it; ++it) {
        if (!mbar_wait_bounded(st_empty, (it & 1) ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) break;
        const int4 item = items[ii];
        const int qt = item_qt(item);
        mbar_expect_tx(st_full, 2 * L::TILE);
#pragma unroll
        for (int db = 0; db < 2; ++db) {
          tma_load_4d_b(sQ + db * SUB, &mapQ, st_full, db * 64, h, qt * BQ, item.x);
          tma_load_4d_b(sDO + db * SUB, &mapdO, st_full, db * 64, h, qt * BQ, item.x);
        }
        if (++ii == nq_it) { ii = 0; ++h; }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one() && n_it > 0) {
      const uint32_t id_s = make_idesc_bf16(128, 64, 0, 0);          // S^T, dP^T of one 64-query half: operands K-major
      const uint32_t id_kv = make_idesc_bf16(128, HD, 0, 1);         // dV, dK: A from TMEM, B = [q rows, d] N-major
      const uint32_t id_q = make_idesc_bf16(128, HD, 1, 1);          // dQ: A = dS^T (M-major), B = K (N-major)
      const uint32_t aK = smem_u32(sK), aV = smem_u32(sV), aQ = smem_u32(sQ), aDO = smem_u32(sDO), aDS = smem_u32(sDS);
      bool ok = mbar_wait_bounded(kv_full, 0, abort_word, p.status, ERR_WAIT_FULL);
      // S^T and dP^T of the 64 queries of half `hf`: contraction over d = 128 (two sub-tiles of four 16-wide steps)
      auto issue_scores = [&](int hf) {
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = (k / 4) * SUB + (k % 4) * 32;
          umma_f16(tmem + C_S, make_smem_desc(aK + ko, 16, 1024), make_smem_desc(aQ + ko + hf * 8192, 16, 1024), id_s, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = (k / 4) * SUB + (k % 4) * 32;
          umma_f16(tmem + C_DP, make_smem_desc(aV + ko, 16, 1024), make_smem_desc(aDO + ko + hf * 8192, 16, 1024), id_s, k ? 1u : 0u);
        }
        umma_commit(&s_full[hf]);
      };
      // dV += P^T dO and dK += dS^T Q over the 64 queries of half `hf` (N = 128: the two d sub-tiles are SUB bytes apart)
      auto issue_kv = [&](int it, int hf) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ts(tmem + C_DV, tmem + C_S + k * 8, make_smem_desc(aDO + hf * 8192 + k * 2048, SUB, 1024), id_kv, (it | hf | k) ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_f16_ts(tmem + C_DK, tmem + C_DP + k * 8, make_smem_desc(aQ + hf * 8192 + k * 2048, SUB, 1024), id_kv, (it | hf | k) ? 1u : 0u);
      };
      for (int it = 0; it < n_it && ok; ++it) {
        if (!mbar_wait_bounded(st_full, it & 1, abort_word, p.status, ERR_WAIT_FULL)) { ok = false; break; }
        tc_fence_after();
        issue_scores(0);
        if (!mbar_wait_bounded(&pds_ready[0], it & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_kv(it, 0);
        issue_scores(1);                                             // reuses the score columns: the pipe runs dV / dK(0) first
        if (!mbar_wait_bounded(&pds_ready[1], it & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        issue_kv(it, 1);
        umma_commit(st_empty);                                       // Q and dO of this step are consumed
        if (!mbar_wait_bounded(dq_empty, (it & 1) ^ 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < BKEY / 16; ++k)                          // contraction over the 128 keys of the block
          umma_f16(tmem + C_DQ, make_smem_desc(aDS + k * 2048, 16384, 1024), make_smem_desc(aK + k * 2048, SUB, 1024), id_q, k ? 1u : 0u);
        umma_commit(dq_full);
      }
      if (ok) umma_commit(acc_final);
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax backward, dQ reduction, dK / dV stores
    const int w = warp - 2;
    const int quarter = warp & 3;
    const int sub = w >> 2;                                  // which CW of a half's 64 query columns
    const int tid = threadIdx.x - 64;
    const int kr = quarter * 32 + lane;                      // key row within the block == TMEM lane
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    constexpr float LOG2E = 1.4426950408889634f;
    bool ok = n_it > 0;
    auto load_aux = [&](const int4& item, int h, float& val, int& e1, int& s2, int& e2) {
      const int qi = item_qt(item) * BQ + (tid & 127);
      const long long base = ((long long)item.x * p.nh + h) * p.Cq;
      if (tid < 128) {
        val = (qi < p.Cq) ? p.lse[base + qi] * LOG2E : 1e30f;
        if (item.y & 1) {                                    // positions relative to this block's first row
          const RowMask rm = item_row_mask(p, item, qi);
          e1 = rm.e1; s2 = rm.s2; e2 = rm.e2;
        }
      } else if (tid < 256) {
        val = (qi < p.Cq) ? p.delta[base + qi] * p.scale : 0.f;
      }
    };
    auto store_aux = [&](int buf, float val, int e1, int s2, int e2) {
      const int x = buf * 128 + (tid & 127);
      if (tid < 128) { sLSE[x] = val; sE1[x] = e1; sS2[x] = s2; sE2[x] = e2; } else if (tid < 256) sDel[x] = val;
    };
    // the dQ tile of step `it` (lanes = queries, 128 columns) goes to global memory 64 columns at a time: TMEM -> shared
    // memory (two [128 x 32] f32 boxes) -> two bulk tensor reductions (f32 add); rows past the sequence end are clipped
    auto reduce_dq = [&](int it, const int4& item, int h) -> bool {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(dq_full, it & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      const int qt = item_qt(item);
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        if (tid == 0) bulk_wait_read0();                     // the previous reduction has finished reading the staging tile
        if (!bar_red_and(3, NM, got)) return false;
        tc_fence_after();
        uint32_t r[CW];
        if constexpr (W16) tmem_ld_32x16(tmem + C_DQ + lane_addr + pass * 64 + sub * CW, r);
        else tmem_ld_32x32(tmem + C_DQ + lane_addr + pass * 64 + sub * CW, r);
        tmem_ld_wait();
        if (pass == 1) { tc_fence_before(); mbar_arrive(dq_empty); }
        // this thread's CW columns lie in box (sub * CW) / 32 at 16-byte piece ((sub * CW) % 32) / 4 of the row
        float* row = sDQ + ((sub * CW) / 32) * (128 * 32) + kr * 32;        // the lane index doubles as the query row here
        const int j0 = ((sub * CW) % 32) / 4;
#pragma unroll
        for (int j = 0; j < CW / 4; ++j)
          *reinterpret_cast<float4*>(row + 4 * ((j0 + j) ^ (kr & 7))) = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                                                      __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
        fence_async_proxy();
        bar_sync_named(2, NM);
        if (tid == 0) {
          tma_reduce_add_4d(&mapdQ, sDQ, pass * 64, h, qt * BQ, item.x);
          tma_reduce_add_4d(&mapdQ, sDQ + 128 * 32, pass * 64 + 32, h, qt * BQ, item.x);
          bulk_commit();
        }
      }
      return true;
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
      int ii_n = ii + 1, h_n = h;                            // the next step's item and head: counters, not divisions
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
#pragma unroll 1
      for (int hf = 0; hf < 2 && ok; ++hf) {
        int got = 1;
        if (lane == 0) got = mbar_wait_bounded(&s_full[hf], it & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        // one verdict for all math warps; at hf == 0 it also publishes this step's LSE / D / mask bounds
        if (!bar_red_and(1, NM, got)) { ok = false; break; }
        tc_fence_after();
        const int c0 = hf * 64 + sub * CW;                   // first query column (within the tile) of this warp in this half
        uint32_t pp[CW / 2], dd[CW / 2];
        {
          uint32_t sr[CW], dr[CW];
          if constexpr (W16) {
            tmem_ld_32x16(tmem + C_S + lane_addr + sub * CW, sr);
            tmem_ld_32x16(tmem + C_DP + lane_addr + sub * CW, dr);
          } else {
            tmem_ld_32x32(tmem + C_S + lane_addr + sub * CW, sr);
            tmem_ld_32x32(tmem + C_DP + lane_addr + sub * CW, dr);
          }
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < CW; i += 4) {
            const float4 l4 = *reinterpret_cast<const float4*>(lse2 + c0 + i);
            const float4 d4 = *reinterpret_cast<const float4*>(del + c0 + i);
            const float lv[4] = {l4.x, l4.y, l4.z, l4.w}, dl[4] = {d4.x, d4.y, d4.z, d4.w};
            float pv[4], dv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              float pe = ex2_approx(fmaf(__uint_as_float(sr[i + u]), sl2, -lv[u]));
              if (need_mask) {
                const int q = c0 + i + u;
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
        }
        // every warp that reads this half's columns has read them: the packed results may now overwrite them
        tc_fence_before();
        bar_sync_named(2, NM);
        tc_fence_after();
        if constexpr (W16) {
          tmem_st_32x8(tmem + C_S + lane_addr + sub * 8, pp);        // 16 queries -> 8 columns of bf16 pairs
          tmem_st_32x8(tmem + C_DP + lane_addr + sub * 8, dd);
        } else {
          tmem_st_32x16(tmem + C_S + lane_addr + sub * 16, pp);      // 32 queries -> 16 columns of bf16 pairs
          tmem_st_32x16(tmem + C_DP + lane_addr + sub * 16, dd);
        }
        {
          // dS^T row kr, queries c0..c0+CW-1, into the M-major A tile: 64-query block hf, 128-byte rows indexed by key
          uint8_t* base = sDS + hf * (128 * 128) + (kr / 8) * 1024 + (kr % 8) * 128;
#pragma unroll
          for (int q = 0; q < CW / 8; ++q)
            *reinterpret_cast<uint4*>(base + (((sub * (CW / 8) + q) ^ (kr % 8)) * 16)) = make_uint4(dd[4 * q], dd[4 * q + 1], dd[4 * q + 2], dd[4 * q + 3]);
        }
        tmem_st_wait();
        fence_async_proxy();
        tc_fence_before();
        mbar_arrive(&pds_ready[hf]);
        if (hf == 0 && it > 0) ok = reduce_dq(it - 1, prev_item, prev_h);     // the previous step's dQ, under this step's products
      }
      if (!ok) break;
      if (it + 1 < n_it) store_aux((it + 1) & 1, vnext, n1, n2, n3);
      prev_item = item; prev_h = h;
      item = next_item; ii = ii_n; h = h_n;
    }
    if (ok) ok = reduce_dq(n_it - 1, prev_item, prev_h);
    if (tid == 0) bulk_wait0();                              // the last dQ reduction has been performed
    // dK, dV of the block: this warp's 64 (W16: 32) of the 128 columns, 32 at a time
    constexpr int OUT_COLS = W16 ? 32 : 64;
    if (ok) {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(acc_final, 0, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got) {
        tc_fence_after();
#pragma unroll 1
        for (int part = 0; part < OUT_COLS / 32; ++part) {
          const int col = sub * OUT_COLS + part * 32;
          uint32_t rv[32], rk[32];
          tmem_ld_32x32(tmem + C_DV + lane_addr + col, rv);
          tmem_ld_32x32(tmem + C_DK + lane_addr + col, rk);
          tmem_ld_wait();
          if (krow + kr < klen) {
            __nv_bfloat16* outK = second ? p.dK2 : p.dK;
            __nv_bfloat16* outV = second ? p.dV2 : p.dV;
            const long long o = (((long long)kseq * klen + krow + kr) * p.nkv + hk) * HD + col;
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
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
      }
    } else if (n_it == 0 && krow + kr < klen) {
      // no query sees this key block: its gradients are zero
      const long long o = (((long long)kseq * klen + krow + kr) * p.nkv + hk) * HD + sub * OUT_COLS;
      const uint4 z = make_uint4(0, 0, 0, 0);
#pragma unroll
      for (int i = 0; i < OUT_COLS; i += 8) {
        *reinterpret_cast<uint4*>((second ? p.dV2 : p.dV) + o + i) = z;
        *reinterpret_cast<uint4*>((second ? p.dK2 : p.dK) + o + i) = z;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

}  // namespace b128

// Called by the entry points of attn_bwd_tcgen05.cu when d == 128; the maps describe 128-wide rows (64-wide boxes, 32 for dQ).
int attn_bwd128_launch(dim3 grid, const CUtensorMap& mq, const CUtensorMap& mdo, const CUtensorMap& mk, const CUtensorMap& mv,
                       const CUtensorMap& mk2, const CUtensorMap& mv2, const CUtensorMap& mdq, const AttnBwdParams& p, const void* O,
                       const void* dO, float* delta, long long q_rows, cudaStream_t stream) {
  using namespace b128;
  delta_kernel<<<(unsigned)((q_rows * 16 + 255) / 256), 256, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(O),
                                                                          reinterpret_cast<const __nv_bfloat16*>(dO), delta, q_rows, p.Cq, p.nh);
  // sixteen math warps unless DTTT_ATTN_BWD_WARPS=8 asks for the eight-warp form
  static const bool sixteen = [] { const char* e = getenv("DTTT_ATTN_BWD_WARPS"); return !(e && e[0] == '8'); }();
  static bool attr = false;
  if (!attr) {
    cudaFuncSetAttribute(attn_bwd128_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    cudaFuncSetAttribute(attn_bwd128_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::TOTAL);
    attr = true;
  }
  if (sixteen) attn_bwd128_kernel<true><<<grid, 576, Smem::TOTAL, stream>>>(mq, mdo, mk, mv, mk2, mv2, mdq, p);
  else attn_bwd128_kernel<false><<<grid, 320, Smem::TOTAL, stream>>>(mq, mdo, mk, mv, mk2, mv2, mdq, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

}  // namespace dttt
