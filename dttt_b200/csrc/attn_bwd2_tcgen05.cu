// Score stage of the second-order attention backward on tcgen05 tensor cores: the four score-shaped products of
// the derivative of the attention backward are formed in tensor memory, reduced along the key axis and turned
// into the four bf16 operand matrices of the output products without ever writing an f32 score to global memory.
// (The reference gets this derivative from JAX differentiating its attention twice, attention.py:181-201.)
//
// With P = softmax(scale Q K^T), dP = dO V^T, D = rowsum(P o dP) and cotangents (gQ, gK, gV) of (dQ, dK, dV):
//   gdS = scale (gQ K^T + Q gK^T)          X = dO gV^T
//   E   = rowsum(P o gdS)                  F = rowsum(P o X) + rowsum(gdS o dS) - E D,   dS = P o (dP - D)
//   out: P,  scale dS,  gdP = P o (gdS - E),  scale gS = scale (P o (X - E dP - F) + gdS o dS)
//
// One CTA = 128 query rows of one (sequence, head); the key axis is swept twice in blocks of 64 keys:
//   warp 0      TMA: the three row tiles (Q, dO, gQ) once, then K, V, gK, gV tiles into a ring of stages
//   warp 1      tcgen05.mma: S, dP, gdS (two products into one accumulator), X into one of two TMEM buffers
//   warps 2-9   one thread per (row, 32-column half): sweep 1 accumulates the three row sums, sweep 2 recomputes
//               the block, writes the four outputs (bf16) into swizzled shared-memory tiles, and one thread
//               stores them with four bulk tensor copies
// The tensor pipe works one block ahead of the arithmetic.  Every wait is bounded; on a timeout all roles leave
// through the common exit and TMEM is freed.
#include "ptx_sm100.cuh"
#include "host_check.h"

#include <mutex>

namespace dttt {

namespace b2 {

constexpr int BQ = 128;    // query rows per CTA
constexpr int BKEY = 64;   // keys per block
constexpr int HD = 64;     // head dimension
constexpr int STAGES = 3;
constexpr int ROW_TILE = BQ * HD * 2;          // 16 KB
constexpr int KEY_TILE = BKEY * HD * 2;        // 8 KB
constexpr int STAGE_BYTES = 4 * KEY_TILE;      // K, V, gK, gV
constexpr int OUT_TILE = BQ * BKEY * 2;        // 16 KB
constexpr int SMEM_TOTAL = 3 * ROW_TILE + STAGES * STAGE_BYTES + 4 * OUT_TILE + 2 * BQ * 3 * 4 + 1024 + 1024;

struct Params {
  int n, Cq, Kn, nh, nkv, causal;
  float scale;
  const float* lse;      // [n, nh, Cq], natural log-sum-exp of the scaled scores
  const float* delta;    // [n, nh, Cq], rowsum(dO o O)
  int* status;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem_src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%2, %3}], [%1];"
               ::"l"(map), "r"(smem_u32(smem_src)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

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

struct Maps {
  CUtensorMap q, dO, gq, k, v, gk, gv, oP, odS, ogdP, ogS;
};

__global__ void __launch_bounds__(320, 1) attn_bwd2_scores_kernel(const __grid_constant__ Maps m, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sDO = sQ + ROW_TILE;
  uint8_t* sGQ = sDO + ROW_TILE;
  uint8_t* sKV = sGQ + ROW_TILE;
  uint8_t* sOut = sKV + STAGES * STAGE_BYTES;                      // four [128 x 64] bf16 tiles, 128-byte swizzle
  float* sStats = reinterpret_cast<float*>(sOut + 4 * OUT_TILE);   // [2 halves][128 rows][3]
  uint64_t* bars = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(sStats) + 2 * BQ * 3 * 4);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + STAGES;
  uint64_t* t_full = kv_empty + STAGES;      // [2]
  uint64_t* t_empty = t_full + 2;            // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(t_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.nh / p.nkv);
  const int q0 = qt * BQ;
  const int nb = p.Kn / BKEY;
  const int n_it = 2 * nb;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&t_full[t], 1); mbar_init(&t_empty[t], 256); }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&m.q); tma_prefetch_desc(&m.dO); tma_prefetch_desc(&m.gq);
    tma_prefetch_desc(&m.k); tma_prefetch_desc(&m.v); tma_prefetch_desc(&m.gk); tma_prefetch_desc(&m.gv);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      mbar_expect_tx(q_full, 3 * ROW_TILE);
      tma_load_4d(sQ, &m.q, q_full, 0, h, q0, b);
      tma_load_4d(sDO, &m.dO, q_full, 0, h, q0, b);
      tma_load_4d(sGQ, &m.gq, q_full, 0, h, q0, b);
      for (int it = 0; it < n_it; ++it) {
        const int s = it % STAGES;
        const int j = it < nb ? it : it - nb;
        if (!mbar_wait_bounded(&kv_empty[s], ((it / STAGES) & 1) ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) break;
        uint8_t* st = sKV + s * STAGE_BYTES;
        mbar_expect_tx(&kv_full[s], STAGE_BYTES);
        tma_load_4d(st, &m.k, &kv_full[s], 0, hk, j * BKEY, b);
        tma_load_4d(st + KEY_TILE, &m.v, &kv_full[s], 0, hk, j * BKEY, b);
        tma_load_4d(st + 2 * KEY_TILE, &m.gk, &kv_full[s], 0, hk, j * BKEY, b);
        tma_load_4d(st + 3 * KEY_TILE, &m.gv, &kv_full[s], 0, hk, j * BKEY, b);
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BQ, BKEY, 0, 0);            // both operands K-major (rows of 64 bf16)
      const uint32_t aQ = smem_u32(sQ), aDO = smem_u32(sDO), aGQ = smem_u32(sGQ);
      bool ok = mbar_wait_bounded(q_full, 0, abort_word, p.status, ERR_WAIT_FULL);
      for (int it = 0; it < n_it && ok; ++it) {
        const int s = it % STAGES, buf = it & 1;
        if (!mbar_wait_bounded(&t_empty[buf], ((it >> 1) & 1) ^ 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) break;
        if (!mbar_wait_bounded(&kv_full[s], (it / STAGES) & 1, abort_word, p.status, ERR_WAIT_FULL)) break;
        tc_fence_after();
        const uint32_t aK = smem_u32(sKV + s * STAGE_BYTES), aV = aK + KEY_TILE, aGK = aK + 2 * KEY_TILE, aGV = aK + 3 * KEY_TILE;
        const uint32_t d0 = tmem + buf * 256;
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = k * 32;                                    // 32 bytes per UMMA_K inside the 128-byte row
          umma_f16(d0, make_smem_desc(aQ + ko, 16, 1024), make_smem_desc(aK + ko, 16, 1024), idesc, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = k * 32;
          umma_f16(d0 + 64, make_smem_desc(aDO + ko, 16, 1024), make_smem_desc(aV + ko, 16, 1024), idesc, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = k * 32;
          umma_f16(d0 + 128, make_smem_desc(aGQ + ko, 16, 1024), make_smem_desc(aK + ko, 16, 1024), idesc, k ? 1u : 0u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = k * 32;
          umma_f16(d0 + 128, make_smem_desc(aQ + ko, 16, 1024), make_smem_desc(aGK + ko, 16, 1024), idesc, 1u);
        }
#pragma unroll
        for (int k = 0; k < HD / 16; ++k) {
          const uint32_t ko = k * 32;
          umma_f16(d0 + 192, make_smem_desc(aDO + ko, 16, 1024), make_smem_desc(aGV + ko, 16, 1024), idesc, k ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(&t_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- row arithmetic: thread = (row, column half)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quarter * 32 + lane;                     // row within the tile == TMEM lane
    const int qi = q0 + row;
    const int tid = threadIdx.x - 64;                        // 0..255
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    constexpr float LOG2E = 1.4426950408889634f;
    const float sl2 = p.scale * LOG2E;
    const long long aux = ((long long)b * p.nh + h) * p.Cq + qi;
    const bool row_ok = qi < p.Cq;
    const float nL2 = row_ok ? -p.lse[aux] * LOG2E : -1e30f;
    const float D = row_ok ? p.delta[aux] : 0.f;
    const int limit = p.causal ? (qi + (p.Kn - p.Cq)) : (p.Kn - 1);     // newest key this row sees
    const long long out_row0 = ((long long)b * p.nh + h) * p.Cq + q0;
    int ok = 1;

    auto wait_block = [&](int it) {
      int got = ok;
      if (ok && lane == 0) got = mbar_wait_bounded(&t_full[it & 1], (it >> 1) & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      ok = got;
      if (ok) tc_fence_after();
    };

    // ---- sweep 1: the three row sums
    float e = 0.f, a = 0.f, bsum = 0.f;
    for (int it = 0; it < nb; ++it) {
      wait_block(it);
      if (ok) {
        const uint32_t t0 = tmem + (it & 1) * 256 + lane_addr + half * 32;
        const int kbase = it * BKEY + half * 32;
#pragma unroll
        for (int c = 0; c < 32; c += 16) {
          uint32_t rs[16], rd[16], rg[16], rx[16];
          tmem_ld_32x16(t0 + c, rs);
          tmem_ld_32x16(t0 + 64 + c, rd);
          tmem_ld_32x16(t0 + 128 + c, rg);
          tmem_ld_32x16(t0 + 192 + c, rx);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float pi = (kbase + c + i <= limit) ? ex2_approx(fmaf(__uint_as_float(rs[i]), sl2, nL2)) : 0.f;
            const float g = __uint_as_float(rg[i]) * p.scale;
            e = fmaf(pi, g, e);
            a = fmaf(pi, __uint_as_float(rx[i]), a);
            bsum = fmaf(g * pi, __uint_as_float(rd[i]) - D, bsum);
          }
        }
        tc_fence_before();
        mbar_arrive(&t_empty[it & 1]);
      }
    }
    sStats[(half * BQ + row) * 3 + 0] = e;
    sStats[(half * BQ + row) * 3 + 1] = a;
    sStats[(half * BQ + row) * 3 + 2] = bsum;
    ok = bar_red_and(1, 256, ok);
    const float E = sStats[row * 3 + 0] + sStats[(BQ + row) * 3 + 0];
    const float F = sStats[row * 3 + 1] + sStats[(BQ + row) * 3 + 1] + sStats[row * 3 + 2] + sStats[(BQ + row) * 3 + 2] - E * D;

    // ---- sweep 2: the four outputs
    uint8_t* my_row = sOut + (row / 8) * 1024 + (row % 8) * 128;       // this row inside a swizzled [128 x 64] bf16 tile
    for (int j = 0; j < nb; ++j) {
      const int it = nb + j;
      wait_block(it);
      // the previous block's stores have finished reading the tiles
      if (tid == 0 && j > 0) bulk_wait_read0();
      ok = bar_red_and(2, 256, ok);
      if (ok) {
        const uint32_t t0 = tmem + (it & 1) * 256 + lane_addr + half * 32;
        const int kbase = j * BKEY + half * 32;
#pragma unroll
        for (int c = 0; c < 32; c += 16) {
          uint32_t rs[16], rd[16], rg[16], rx[16];
          tmem_ld_32x16(t0 + c, rs);
          tmem_ld_32x16(t0 + 64 + c, rd);
          tmem_ld_32x16(t0 + 128 + c, rg);
          tmem_ld_32x16(t0 + 192 + c, rx);
          tmem_ld_wait();
          uint32_t oP[8], oS[8], oG[8], oX[8];
#pragma unroll
          for (int i = 0; i < 16; i += 2) {
            float vP[2], vS[2], vG[2], vX[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
              const float pi = (kbase + c + i + u <= limit) ? ex2_approx(fmaf(__uint_as_float(rs[i + u]), sl2, nL2)) : 0.f;
              const float g = __uint_as_float(rg[i + u]) * p.scale;
              const float dp = __uint_as_float(rd[i + u]);
              const float ds = pi * (dp - D);
              vP[u] = pi;
              vS[u] = ds * p.scale;
              vG[u] = pi * (g - E);
              vX[u] = (fmaf(pi, __uint_as_float(rx[i + u]) - fmaf(E, dp, F), g * ds)) * p.scale;
            }
            __nv_bfloat162 t;
            t = __floats2bfloat162_rn(vP[0], vP[1]); oP[i / 2] = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2bfloat162_rn(vS[0], vS[1]); oS[i / 2] = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2bfloat162_rn(vG[0], vG[1]); oG[i / 2] = *reinterpret_cast<uint32_t*>(&t);
            t = __floats2bfloat162_rn(vX[0], vX[1]); oX[i / 2] = *reinterpret_cast<uint32_t*>(&t);
          }
          // 16 columns = two 16-byte chunks of this row in each tile
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int chunk = (half * 32 + c) / 8 + q;
            const int off = (chunk ^ (row % 8)) * 16;
            *reinterpret_cast<uint4*>(my_row + off) = make_uint4(oP[4 * q], oP[4 * q + 1], oP[4 * q + 2], oP[4 * q + 3]);
            *reinterpret_cast<uint4*>(my_row + OUT_TILE + off) = make_uint4(oS[4 * q], oS[4 * q + 1], oS[4 * q + 2], oS[4 * q + 3]);
            *reinterpret_cast<uint4*>(my_row + 2 * OUT_TILE + off) = make_uint4(oG[4 * q], oG[4 * q + 1], oG[4 * q + 2], oG[4 * q + 3]);
            *reinterpret_cast<uint4*>(my_row + 3 * OUT_TILE + off) = make_uint4(oX[4 * q], oX[4 * q + 1], oX[4 * q + 2], oX[4 * q + 3]);
          }
        }
        tc_fence_before();
        mbar_arrive(&t_empty[it & 1]);
        fence_async_proxy();
      }
      ok = bar_red_and(3, 256, ok);
      if (ok && tid == 0) {
        const int x = j * BKEY, y = (int)out_row0;
        tma_store_2d(&m.oP, sOut, x, y);
        tma_store_2d(&m.odS, sOut + OUT_TILE, x, y);
        tma_store_2d(&m.ogdP, sOut + 2 * OUT_TILE, x, y);
        tma_store_2d(&m.ogS, sOut + 3 * OUT_TILE, x, y);
        bulk_commit();
      }
    }
    if (tid == 0) bulk_wait0();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// bf16 [n, rows, heads, 64] contiguous; box = 64 x 1 head x box_rows x 1, 128-byte swizzle
static int make_in_map(CUtensorMap* map, const void* ptr, int n, int rows, int heads, int box_rows) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[4] = {(cuuint64_t)HD, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)HD * 2, (cuuint64_t)heads * HD * 2, (cuuint64_t)rows * heads * HD * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (int c = check_map(ptr, 4, dims, strides, 2)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// bf16 [rows, Kn] contiguous; box = 64 columns x 128 rows, 128-byte swizzle
static int make_out_map(CUtensorMap* map, void* ptr, long long rows, int Kn) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)Kn, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)Kn * 2};
  cuuint32_t box[2] = {BKEY, BQ};
  cuuint32_t estr[2] = {1, 1};
  if (int c = check_map(ptr, 2, dims, strides, 2)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace b2
}  // namespace dttt

using namespace dttt;

// Q, dO, gQ [n, Cq, nh, 64]; K, V, gK, gV [n, Kn, nkv, 64] (bf16, contiguous); lse, delta [n, nh, Cq] f32;
// outputs P, dS, gdP, gS: bf16 [n * nh * Cq, Kn] (row = (b * nh + h) * Cq + i), dS and gS pre-multiplied by `scale`.
// Cq a multiple of 128, Kn a multiple of 64; `causal` aligns the triangle to the end of the key axis.
// Returns 0, -1 for an unsupported shape, another value for a failed set-up step.
extern "C" int dttt_attn_bwd2_scores(const void* Q, const void* dO, const void* gQ, const void* K, const void* V, const void* gK,
                                     const void* gV, const float* lse, const float* delta, void* P, void* dS, void* gdP, void* gS,
                                     int n, int Cq, int Kn, int nh, int nkv, float scale, int causal, int* status, void* stream) {
  if (n <= 0 || Cq <= 0 || Cq % b2::BQ || Kn <= 0 || Kn % b2::BKEY || nkv <= 0 || nh % nkv) return -1;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { cudaFree(0); ctx_bound = true; }
  b2::Maps m;
  int r;
  if ((r = b2::make_in_map(&m.q, Q, n, Cq, nh, b2::BQ))) return 100 + r;
  if ((r = b2::make_in_map(&m.dO, dO, n, Cq, nh, b2::BQ))) return 200 + r;
  if ((r = b2::make_in_map(&m.gq, gQ, n, Cq, nh, b2::BQ))) return 300 + r;
  if ((r = b2::make_in_map(&m.k, K, n, Kn, nkv, b2::BKEY))) return 400 + r;
  if ((r = b2::make_in_map(&m.v, V, n, Kn, nkv, b2::BKEY))) return 500 + r;
  if ((r = b2::make_in_map(&m.gk, gK, n, Kn, nkv, b2::BKEY))) return 600 + r;
  if ((r = b2::make_in_map(&m.gv, gV, n, Kn, nkv, b2::BKEY))) return 700 + r;
  const long long rows = (long long)n * nh * Cq;
  if ((r = b2::make_out_map(&m.oP, P, rows, Kn))) return 800 + r;
  if ((r = b2::make_out_map(&m.odS, dS, rows, Kn))) return 900 + r;
  if ((r = b2::make_out_map(&m.ogdP, gdP, rows, Kn))) return 1000 + r;
  if ((r = b2::make_out_map(&m.ogS, gS, rows, Kn))) return 1100 + r;
  b2::Params p;
  p.n = n; p.Cq = Cq; p.Kn = Kn; p.nh = nh; p.nkv = nkv; p.causal = causal; p.scale = scale;
  p.lse = lse; p.delta = delta; p.status = status;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(b2::attn_bwd2_scores_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, b2::SMEM_TOTAL) != cudaSuccess) return 1200;
    attr = true;
  }
  dim3 grid(Cq / b2::BQ, nh, n);
  b2::attn_bwd2_scores_kernel<<<grid, 320, b2::SMEM_TOTAL, (cudaStream_t)stream>>>(m, p);
  return (int)cudaGetLastError();
}
