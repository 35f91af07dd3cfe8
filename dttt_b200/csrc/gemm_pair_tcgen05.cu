// bf16 GEMM on CTA PAIRS: two CTAs of a cluster compute one 256 x 256 output tile with tcgen05.mma.cta_group::2.
//
//   C[b] (+)= alpha * A[b] x B[b]          (same operand conventions as gemm_tcgen05.cu)
//
// Why pairs.  With one CTA per 128 x 256 tile every k-block moves (128 + 256) x 64 bf16 = 48 KB from L2 into shared memory
// for 128 x 256 x 64 multiply-adds; on the model's shapes (K = 2048, weights shared by every row tile) that traffic, not the
// tensor pipe, sets the pace.  A pair splits B: each CTA loads its own 128 rows of A and HALF of the 256 B columns, the
// instruction reads both halves, and each CTA still accumulates a full 128 x 256 tile in its own tensor memory: 32 KB per CTA
// and k-block for the same math, with the two-accumulator overlap of epilogue and main loop kept (512 TMEM columns per CTA).
//
// No load is multicast: each CTA issues plain per-CTA TMA loads of its own halves.  What crosses the pair is
//   * the "stage is full" count: both CTAs' loads complete on the LEADER's mbarrier (cp.async.bulk.tensor.cta_group::2),
//   * the instruction itself (issued by one thread of the leader, cluster rank 0),
//   * tcgen05.commit arriving on the "stage free" / "accumulator ready" barriers of BOTH CTAs,
//   * the follower's epilogue threads arriving on the leader's "accumulator drained" barrier.
// Every wait is bounded; a CTA that gives up sets the status word, and its partner's waits then run out the same way.
#include "ptx_sm100.cuh"
#include "host_check.h"

#include <cstdlib>
#include <cstring>
#include <mutex>

namespace dttt {
namespace pair {

constexpr int BM = 128;        // rows of A per CTA (256 per pair)
constexpr int BN = 256;        // output columns per pair; each CTA loads BN / 2 of them
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK * 2;
constexpr int B_BYTES = (BN / 2) * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;                 // 32 KB per CTA
constexpr int STAGING_BYTES = 4 * 4096;                        // epilogue: 32 rows x 128 bytes per warp (whole-line stores)
constexpr int SMEM_TOTAL = STAGES * STAGE_BYTES + 1024 + STAGING_BYTES + 1024;

struct Params {
  int M, N, K, batch;
  int a_mn_major, b_mn_major;
  long long ldc, c_batch;
  int c_is_f32, accumulate;
  int per_lane_stores;         // 1: 16 bytes per lane and row instead of whole lines (DTTT_GEMM_LINES=0; for comparisons)
  float alpha;
  void* C;
  int* status;
  int tiles_m, tiles_n;        // pair tiles: 256 x 256
};

__device__ __forceinline__ void tile_coords(int tile, const Params& p, int& b, int& tm, int& tn) {
  const int per_batch = p.tiles_m * p.tiles_n;
  b = tile / per_batch;
  const int t = tile - b * per_batch;
  constexpr int GROUP = 8;                                     // bands of 8 pair rows, n fastest inside a band
  const int band = t / (GROUP * p.tiles_n);
  const int first_m = band * GROUP;
  const int rows = min(GROUP, p.tiles_m - first_m);
  const int r = t - band * GROUP * p.tiles_n;
  tm = first_m + (r % rows);
  tn = r / rows;
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(192, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + STAGES * STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);      // leader's are used: bytes of BOTH CTAs land there
  uint64_t* empty = full + STAGES;                             // per CTA: its stage may be overwritten
  uint64_t* acc_full = empty + STAGES;                         // per CTA: its accumulator half is complete
  uint64_t* acc_empty = acc_full + 2;                          // leader's are used: both CTAs' epilogues have drained it
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                     // 0 = leader
  const int pair_id = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int num_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 256); }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
  }
  if (warp == 1) {                                             // one warp of EACH CTA takes part in the pair's allocation
    tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                                          // both CTAs' barriers exist and both have their tensor memory
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (each CTA loads its own halves)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += n_pairs) {
        int b, tm, tn;
        tile_coords(tile, p, b, tm, tn);
        const int m0 = tm * 2 * BM + (int)rank * BM;
        const int n0 = tn * BN + (int)rank * (BN / 2);
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded(&empty[s], ph ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + s * STAGE_BYTES;
          uint8_t* sB = sA + A_BYTES;
          if (rank == 0) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);     // this CTA's bytes and the partner's
          const uint32_t bar = mapa_u32(&full[s], 0);                   // the leader's barrier, from either CTA
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_3d_pair(sA, &mapA, bar, k0, m0, b);                // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_3d_pair(sA + j * (BK * 128), &mapA, bar, m0 + j * 64, k0, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d_pair(sB, &mapB, bar, k0, n0, b);                // box {64 k, 128 rows of B}
          } else {
#pragma unroll
            for (int j = 0; j < (BN / 2) / 64; ++j) tma_load_3d_pair(sB + j * (BK * 128), &mapB, bar, n0 + j * 64, k0, b);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (rank == 0 && elect_one()) {
      const uint32_t idesc = make_idesc_bf16(2 * BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += n_pairs, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[acc], acc_ph ^ 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait_bounded(&full[s], ph, abort_word, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sB = sA + A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_pair(d_tmem, make_smem_desc(sA + k * a_kstep, a_lbo, 1024), make_smem_desc(sB + k * b_kstep, b_lbo, 1024), idesc,
                          (kb | k) ? 1u : 0u);
          umma_commit_pair(&empty[s], 3);                      // frees the stage in BOTH CTAs once these MMAs have read it
        }
        if (ok) umma_commit_pair(&acc_full[acc], 3);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5 of each CTA: its own 128 rows)
    const int quarter = warp & 3;
    uint32_t local_tile = 0;
    for (int tile = pair_id; tile < num_tiles; tile += n_pairs, ++local_tile) {
      int b, tm, tn;
      tile_coords(tile, p, b, tm, tn);
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(&acc_full[acc], acc_ph, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      const int row = tm * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      const long long row_off = (long long)b * p.c_batch + (long long)row * p.ldc;
      // stores and reductions as whole 128-byte lines (warp-uniform conditions; ragged column edges, odd strides and bf16
      // accumulation take the per-lane path below)
      const bool lines16 = !p.per_lane_stores && !p.c_is_f32 && !p.accumulate && (p.ldc & 7) == 0 &&
                           ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_batch * 2)) & 15) == 0;
      const bool lines32 = !p.per_lane_stores && p.c_is_f32 && (p.ldc & 3) == 0 &&
                           ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_batch * 4)) & 15) == 0;
      uint8_t* stg = bar_base + 1024 + quarter * 4096;
      const int row0 = tm * 2 * BM + (int)rank * BM + quarter * 32;
      const long long tile_off = (long long)b * p.c_batch + (long long)row0 * p.ldc + n0;
      const float alpha = p.alpha;
      auto scale = [alpha](float v, int) { return v * alpha; };
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (lines16 && (c & 32) == 0 && n0 + c + 64 <= p.N) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c, r0);
          tmem_ld_32x32(taddr + c + 32, r1);
          tmem_ld_wait();
          stage_put_bf16x32(stg, lane, 0, r0, scale);
          stage_put_bf16x32(stg, lane, 1, r1, scale);
          __syncwarp();
          stage_flush_bf16x64(stg, lane, reinterpret_cast<__nv_bfloat16*>(p.C) + tile_off + c, p.ldc, p.M - row0);
          __syncwarp();
          c += 32;
          continue;
        }
        if (lines32 && n0 + c + 32 <= p.N) {
          uint32_t r0[32];
          tmem_ld_32x32(taddr + c, r0);
          tmem_ld_wait();
          stage_put_f32x32(stg, lane, r0, scale);
          __syncwarp();
          stage_flush_f32x32(stg, lane, reinterpret_cast<float*>(p.C) + tile_off + c, p.ldc, p.M - row0, p.accumulate != 0);
          __syncwarp();
          continue;
        }
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
        const int col = n0 + c;
        if (row_ok && col < p.N) {
          const bool full_chunk = (col + 32 <= p.N);
          if (p.c_is_f32) {
            float* out = reinterpret_cast<float*>(p.C) + row_off + col;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 v = make_float4(__uint_as_float(r[j]) * p.alpha, __uint_as_float(r[j + 1]) * p.alpha,
                                       __uint_as_float(r[j + 2]) * p.alpha, __uint_as_float(r[j + 3]) * p.alpha);
                if (p.accumulate) red_add_f32x4(out + j, v);       // C += tile as a vector reduction at L2 (no load to wait for)
                else *reinterpret_cast<float4*>(out + j) = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float v = __uint_as_float(r[j]) * p.alpha;
                if (p.accumulate) v += out[j];
                out[j] = v;
              }
            }
          } else {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + row_off + col;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float f[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) f[q] = __uint_as_float(r[j + q]) * p.alpha;
                if (p.accumulate) {
                  const uint4 o = *reinterpret_cast<uint4*>(out + j);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    const float2 of = __bfloat1622float2(ob[q]);
                    f[2 * q] += of.x; f[2 * q + 1] += of.y;
                  }
                }
                uint4 v;
                __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                for (int q = 0; q < 4; ++q) vb[q] = __floats2bfloat162_rn(f[2 * q], f[2 * q + 1]);
                *reinterpret_cast<uint4*>(out + j) = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float v = __uint_as_float(r[j]) * p.alpha;
                if (p.accumulate) v += __bfloat162float(out[j]);
                out[j] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      tc_fence_before();
      // this CTA's half of accumulator `acc` is drained: tell the leader (128 threads of each CTA -> 256 arrivals)
      mbar_arrive_remote(mapa_u32(&acc_empty[acc], 0));
    }
  }

  // ---------------------------------------------------------------- common exit: nobody leaves while the partner may still reach in
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
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

static int make_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long batch, long long outer_stride_elems,
                    long long batch_stride_elems, int box_outer) {
  EncodeTiledFn enc = encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)outer_stride_elems * 2, (cuuint64_t)(batch > 1 ? batch_stride_elems : outer_stride_elems * outer) * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if (int c = check_map(ptr, 3, dims, strides, 2)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace pair
}  // namespace dttt

// The GEMM of dttt_gemm_bf16 on CTA pairs.  Arguments as there (without max_ctas).  Returns 0 on a clean launch.
extern "C" int dttt_gemm_pair_bf16(const void* A, const void* B, void* C, int M, int N, int K, int batch, long long lda, long long ldb,
                                   long long ldc, long long a_batch, long long b_batch, long long c_batch, int a_mn_major, int b_mn_major,
                                   int c_is_f32, int accumulate, float alpha, int* status, cudaStream_t stream) {
  using namespace dttt::pair;
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) || (a_batch % 8) || (b_batch % 8))
    return -2;
  static thread_local int bound_dev = -1;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return -3;
  if (bound_dev != dev) { cudaSetDevice(dev); cudaFree(0); bound_dev = dev; }
  CUtensorMap mapA, mapB;
  int r;
  if (!a_mn_major) r = make_map(&mapA, A, K, M, batch, lda, a_batch, BM);
  else             r = make_map(&mapA, A, M, K, batch, lda, a_batch, BK);
  if (r) return 100 + r;
  if (!b_mn_major) r = make_map(&mapB, B, K, N, batch, ldb, b_batch, BN / 2);
  else             r = make_map(&mapB, B, N, K, batch, ldb, b_batch, BK);
  if (r) return 200 + r;
  Params p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.batch = batch; p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.ldc = ldc; p.c_batch = c_batch; p.c_is_f32 = c_is_f32; p.accumulate = accumulate; p.alpha = alpha; p.C = C; p.status = status;
  { static const int per_lane = (getenv("DTTT_GEMM_LINES") && atoi(getenv("DTTT_GEMM_LINES")) == 0) ? 1 : 0; p.per_lane_stores = per_lane; }
  p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
  p.tiles_n = (N + BN - 1) / BN;
  static std::mutex mu;
  static unsigned long long attr_mask = 0;
  static int sms[64] = {0};
  {
    std::lock_guard<std::mutex> lock(mu);
    if (dev >= 0 && dev < 64) {
      if (!(attr_mask >> dev & 1ull)) {
        cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_TOTAL);
        cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
        attr_mask |= 1ull << dev;
      }
    }
  }
  const int n_sm = (dev >= 0 && dev < 64 && sms[dev] > 0) ? sms[dev] : 148;
  const long long tiles = (long long)batch * p.tiles_m * p.tiles_n;
  const int pairs = (int)(tiles < n_sm / 2 ? tiles : n_sm / 2);
  gemm_pair_kernel<<<2 * pairs, 192, SMEM_TOTAL, stream>>>(mapA, mapB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
