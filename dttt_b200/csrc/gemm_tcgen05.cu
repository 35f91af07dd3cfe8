// Persistent, warp-specialised bf16 GEMM for sm_100a: TMA -> shared memory (128B swizzle) ->
// tcgen05.mma with the f32 accumulator in tensor memory -> tcgen05.ld epilogue.
//
//   C[b] (+)= alpha * A[b] x B[b]      A: M x K,  B: K x N,  C: M x N (row-major, bf16 or f32)
//
// Either operand may be stored K-major (contraction index contiguous) or MN-major (the M / N index
// contiguous); all four combinations run on the tensor core without a transpose pass, which is
// what lets one kernel serve y = x @ W, dx = dy @ W^T and dW = x^T @ dy for weights stored
// [in, out] (the layout of reference src/ttt/model.py:137-148).  A leading batch index (a 3-D
// tensor map) gives the per-sequence fast-weight products (reference model.py:316-319, one weight
// per sequence) in one launch.
//
// Roles of the 192 threads of a CTA (one CTA per SM, grid = min(tiles, SMs)):
//   warp 0     TMA producer   (one elected lane)
//   warp 1     MMA issuer     (one elected lane) and TMEM owner
//   warps 2-5  epilogue       (TMEM lane quarter = warp index % 4)
// Two accumulators of BN columns alternate so the epilogue of tile i overlaps the main loop of
// tile i+1.  Every wait is bounded (ptx_sm100.cuh); on a timeout all roles leave through the
// common exit, the status word says which wait gave up and TMEM is freed.
#include "ptx_sm100.cuh"
#include "host_check.h"

#include <mutex>
#include <unordered_map>
#include <cstring>
#include <cstdio>
#include <cstdlib>

namespace dttt {

constexpr int BM = 128;
constexpr int BK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int UMMA_K = 16;

#define DTTT_MAX_TP 8

struct GemmParams {
  int M, N, K, batch;
  int a_mn_major, b_mn_major;
  long long ldc;        // elements
  long long c_batch;    // elements
  int c_is_f32;
  int per_lane_stores;  // 1: the bf16 store epilogue writes 16 bytes per lane and row (DTTT_GEMM_LINES=0; for comparisons)
  int accumulate;       // C += result
  float alpha;
  void* C;
  int* status;
  int tiles_m, tiles_n;
  // cross-entropy epilogues (MODE 1 / 2)
  const int* targets;       // [M] class index of every row (columns are classes, offset by col0)
  const float* row_coef;    // [M] MODE 2: g * w_row
  const float* row_lse;     // [M] MODE 2: log-partition of the row
  float2* part;             // MODE 1: [tiles_n][part_stride] per-tile (max, sum exp(x - max))
  float* tgt_logit;         // MODE 1: [M] logit of the target class
  long long part_stride;
  int col0;                 // class index of column 0
  // fused collectives (MODE 3 / 4): one process per GPU, every pointer below is valid on THIS GPU (CUDA IPC)
  int m_rotate;             // tile rows are visited starting at this m-block (own rows first)
  int tp, self_rank, epoch;
  int rows_per_rank;        // M / tp, a multiple of BM
  long long a_row_bytes;    // MODE 3: bytes of one row of A that carry data (K * 2)
  long long lda_bytes;      // MODE 3: row stride of the gather buffer in bytes
  void* peer_a[DTTT_MAX_TP];      // MODE 3: rank r's gather buffer [M, K] (entry self_rank is the local one)
  int* peer_flags[DTTT_MAX_TP];   // rank r's flag words: [0, tp) "shard of rank s is in place", [tp, 2 tp) "partials of rank s have landed"
  int* ready;               // MODE 3: local [tiles_m] words, epoch of the last completed copy of that m-block
  // MODE 5: the weight (the B operand, [wg_rows, wg_row_elems] bf16, dense) is gathered from the ranks' flat shards: element e of
  // the flat parameter space lives at peer_a[e / wg_shard_elems] + (e % wg_shard_elems); `ready` has one word per 64 weight rows
  int n_rotate;             // tile columns are visited starting at this n-block
  int wg_on_k;              // 0: weight rows are output columns (K-major B); 1: weight rows are the contraction index (N-major B)
  int wg_rows, wg_rot;      // rows of the weight; 64-row block the copies (and the visiting order) start at
  long long wg_flat_off;    // flat index of the weight's first element
  long long wg_shard_elems; // elements of the flat space per rank
  long long wg_row_elems;   // elements per weight row
  void* wg_dst;             // local dense copy of the weight that the TMA reads
  int wg_parts;             // CTAs that share the copy of one 64-row block (so every CTA's copy warps pull something)
  int* wg_cnt;              // per block: parts finished so far in this launch (the last one resets it and raises the ready word)
  void* peer_c[DTTT_MAX_TP];      // MODE 4: rank r's slot buffer [tp][rows_per_rank][N] bf16
  int* done_counter;        // MODE 4: local CTA counter, never reset
  int done_target;          // MODE 4: its value once every CTA of this launch has finished
};

// Epilogue modes of the kernel below.
//   0  C (+)= alpha * acc                                           (the GEMM)
//   1  no C: per row and column tile, (max, sum exp) of the tile's logits and the target's logit
//      (the forward of linear + cross-entropy, reference src/ttt/fused_ce.py:42-73)
//   2  C = coef[row] * (exp(acc - lse[row]) - [col == target[row]])  in bf16
//      (d loss / d logits, reference fused_ce.py:93-104), consumed by the two gradient GEMMs
//   3  the GEMM with the all-gather of A fused in: rows of A owned by other ranks are pulled from their memory over
//      NVLink by four copy warps per CTA into the local gather buffer while the tensor core works on the rows that
//      are already here; the TMA producer waits (bounded) on a per-m-block ready word before touching a pulled block
//   4  the GEMM with the reduce-scatter of C fused in: every finished tile is stored straight into the slot
//      [this rank] of the rank that owns those rows; the last CTA to finish raises this rank's flag at every peer
//   5  the GEMM with the all-gather of a sharded WEIGHT (the B operand) fused in: four copy warps per CTA pull the weight,
//      64 rows at a time, from the flat parameter shards of the ranks that own them (peer loads over NVLink, the own part
//      from local memory) into a dense local buffer; the TMA producer waits (bounded) on the ready words of the rows a
//      tile (or, when the weight's rows are the contraction index, a k-block) needs.  Tiles and k-blocks are visited
//      starting at the block the copies start at.  The shards must not change while any rank runs the kernel
//      (the optimiser step is separated from the passes by collectives).
constexpr int EPI_STORE = 0, EPI_CE_PARTIAL = 1, EPI_CE_DLOGITS = 2, EPI_AG = 3, EPI_RS = 4, EPI_WG = 5;
constexpr int WG_ROWS = 64;

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
  int v;
  asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
  asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
// Barrier `id` over 128 threads that also ANDs a per-thread flag (one verdict for the four copy warps).
__device__ __forceinline__ int bar_red_and_128(int id, int flag) {
  int out;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, %2, 128, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t}"
      : "=r"(out) : "r"(flag), "r"(id) : "memory");
  return out;
}
// Spin until *flag >= target, for at most a second; on a timeout record `err` and raise the CTA's abort word.
template <bool SYS>
__device__ __forceinline__ bool wait_flag_ge(const int* flag, int target, volatile int* abort_word, int* status, int err) {
  const uint64_t t0 = global_timer_ns();
  uint32_t spins = 0;
  while (true) {
    const int v = SYS ? ld_acquire_sys(flag) : ld_acquire_gpu(flag);
    if (v - target >= 0) return true;
    if (*abort_word) return false;
    if ((++spins & 63u) == 0 && global_timer_ns() - t0 > 1000000000ull) {
      *abort_word = 1;
      if (status) atomicCAS(status, 0, err);
      return false;
    }
    __nanosleep(64);
  }
}


template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int BAR_BYTES = 1024;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
  // EPI_RS stages finished tiles through shared memory so rows leave in 256-byte pieces: 4 warps x 32 rows x 128 columns
  static constexpr int RS_STAGE_BYTES = 4 * 32 * 128 * 2;
  static constexpr int TOTAL_RS = TOTAL + RS_STAGE_BYTES;
};

__device__ __forceinline__ void tile_coords(int tile, const GemmParams& p, int& b, int& tm, int& tn) {
  int per_batch = p.tiles_m * p.tiles_n;
  b = tile / per_batch;
  int t = tile - b * per_batch;
  // Bands of 16 m-tiles, n fastest inside a band: concurrently running CTAs share A rows and sweep B.
  constexpr int GROUP = 16;
  int band = t / (GROUP * p.tiles_n);
  int first_m = band * GROUP;
  int rows = min(GROUP, p.tiles_m - first_m);
  int r = t - band * GROUP * p.tiles_n;
  tm = first_m + (r % rows);
  tn = r / rows;
  if (p.m_rotate) tm = (tm + p.m_rotate) % p.tiles_m;
  if (p.n_rotate) tn = (tn + p.n_rotate) % p.tiles_n;
}

template <int BN, int MODE>
__global__ void __launch_bounds__((MODE == EPI_AG || MODE == EPI_WG) ? 320 : 192, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
                 const GemmParams p) {
  using L = SmemLayout<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + L::STAGES * L::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty = full + L::STAGES;
  uint64_t* acc_full = empty + L::STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // 256 or 512: a power of two >= 32

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], 1); mbar_init(&acc_empty[a], 128); }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, tm, tn;
        tile_coords(tile, p, b, tm, tn);
        const int m0 = tm * BM, n0 = tn * BN;
        if constexpr (MODE == EPI_AG) {
          // rows pulled from another rank: wait until the copy warps (of whichever CTA took that block) have
          // finished it; their stores were generic-proxy writes, the loads below go through the async proxy
          if (m0 / p.rows_per_rank != p.self_rank) {
            if (!wait_flag_ge<false>(p.ready + tm, p.epoch, abort_word, p.status, ERR_WAIT_PEER)) { ok = false; break; }
            fence_async_proxy();
          }
        }
        if constexpr (MODE == EPI_WG) {
          if (!p.wg_on_k) {
            // the weight rows of this tile's columns: wait for the copy warps (of whichever CTAs took those blocks)
            const int nblk = (p.wg_rows + WG_ROWS - 1) / WG_ROWS;
            for (int j = 0; j < BN / WG_ROWS && ok; ++j) {
              const int blk = n0 / WG_ROWS + j;
              if (blk < nblk && !wait_flag_ge<false>(p.ready + blk, p.epoch, abort_word, p.status, ERR_WAIT_PEER)) ok = false;
            }
            if (!ok) break;
            fence_async_proxy();
          }
        }
        for (int kb_ = 0; kb_ < kblocks; ++kb_, ++it) {
          int kb = kb_;
          if constexpr (MODE == EPI_WG) {
            if (p.wg_on_k) {
              // k-blocks are 64 weight rows each: start at the block the copies start at; after this CTA's first tile
              // every block has been seen ready
              kb = kb_ + p.wg_rot;
              if (kb >= kblocks) kb -= kblocks;
              if (tile == (int)blockIdx.x) {
                if (!wait_flag_ge<false>(p.ready + kb, p.epoch, abort_word, p.status, ERR_WAIT_PEER)) { ok = false; break; }
                fence_async_proxy();
              }
            }
          }
          const int s = it % L::STAGES;
          const uint32_t ph = (it / L::STAGES) & 1;
          if (!mbar_wait_bounded(&empty[s], ph ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_3d(sA, &mapA, &full[s], k0, m0, b);                 // box {64 k, 128 rows}
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j)                            // box {64 m, 64 k-rows}
              tma_load_3d(sA + j * (BK * 128), &mapA, &full[s], m0 + j * 64, k0, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d(sB, &mapB, &full[s], k0, n0, b);                 // box {64 k, BN rows}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * (BK * 128), &mapB, &full[s], n0 + j * 64, k0, b);
          }
        }
      }
      if (!ok) {
        // Unwinding: give the copies already issued a bounded time to land before the CTA exits.
        // (Every issued stage either completed its full barrier or is about to; nothing to free.)
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;   // bytes per UMMA_K
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const int acc = local_tile & 1;
        const uint32_t acc_ph = (local_tile >> 1) & 1;
        if (!mbar_wait_bounded(&acc_empty[acc], acc_ph ^ 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t ph = (it / L::STAGES) & 1;
          if (!mbar_wait_bounded(&full[s], ph, abort_word, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t ad = make_smem_desc(sA + k * a_kstep, a_lbo, 1024);
            const uint64_t bd = make_smem_desc(sB + k * b_kstep, b_lbo, 1024);
            umma_f16(d_tmem, ad, bd, idesc, (kb | k) ? 1u : 0u);
          }
          umma_commit(&empty[s]);      // frees the stage once these MMAs have read it
        }
        if (ok) umma_commit(&acc_full[acc]);
      }
    }
    __syncwarp();
  } else if (warp >= 6) {
    // ------------------------------------------------------------ copy warps (MODE 3 only): the all-gather
    if constexpr (MODE == EPI_AG) {
      const int ct = threadIdx.x - 192;                              // 0..127
      if (blockIdx.x == 0 && ct < p.tp) st_release_sys(p.peer_flags[ct] + p.self_rank, p.epoch);   // my shard is in place
      const int bpr = p.rows_per_rank / BM;                          // m-blocks per rank
      const int n_remote = p.tiles_m - bpr;
      const int vec_per_row = (int)(p.a_row_bytes / 16);
      const int total = BM * vec_per_row;
      for (int i = blockIdx.x; i < n_remote; i += gridDim.x) {
        const int tm = (bpr + i + p.self_rank * bpr) % p.tiles_m;     // the order the tiles are visited in
        const int src = tm / bpr;
        int got = 1;
        if (lane == 0) got = wait_flag_ge<true>(p.peer_flags[p.self_rank] + src, p.epoch, abort_word, p.status, ERR_WAIT_PEER) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!bar_red_and_128(4, got)) break;
        const char* from = reinterpret_cast<const char*>(p.peer_a[src]) + (long long)tm * BM * p.lda_bytes;
        char* to = reinterpret_cast<char*>(p.peer_a[p.self_rank]) + (long long)tm * BM * p.lda_bytes;
        for (int v0 = ct; v0 < total; v0 += 128 * 8) {
          uint4 buf[8];
          long long offs[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const int idx = v0 + u * 128;
            const int row = idx / vec_per_row, col = idx - row * vec_per_row;
            offs[u] = (long long)row * p.lda_bytes + (long long)col * 16;
            if (idx < total) buf[u] = ld_relaxed_sys_v4(from + offs[u]);
          }
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v0 + u * 128 < total) *reinterpret_cast<uint4*>(to + offs[u]) = buf[u];
        }
        __threadfence();
        asm volatile("bar.sync 4, 128;" ::: "memory");
        if (ct == 0) { fence_async_proxy(); st_release_gpu(p.ready + tm, p.epoch); }
      }
    }
    if constexpr (MODE == EPI_WG) {
      const int ct = threadIdx.x - 192;                              // 0..127
      const int nblk = (p.wg_rows + WG_ROWS - 1) / WG_ROWS;
      const long long vec_per_blk = (long long)WG_ROWS * p.wg_row_elems / 8;
      const long long vec_total = (long long)p.wg_rows * p.wg_row_elems / 8;
      const long long shard_vecs = p.wg_shard_elems / 8, flat0 = p.wg_flat_off / 8;
      const long long vec_per_part = (vec_per_blk + p.wg_parts - 1) / p.wg_parts;
      for (int i = blockIdx.x; i < nblk * p.wg_parts; i += gridDim.x) {
        int blk = i / p.wg_parts + p.wg_rot;
        const int part = i % p.wg_parts;
        if (blk >= nblk) blk -= nblk;
        const long long b_lo = (long long)blk * vec_per_blk;
        const long long v_lo = b_lo + part * vec_per_part;
        const long long v_hi = min(min(v_lo + vec_per_part, b_lo + vec_per_blk), vec_total);
        uint4* to = reinterpret_cast<uint4*>(p.wg_dst);
        for (long long v0 = v_lo + ct; v0 < v_hi; v0 += 128 * 8) {
          uint4 buf[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const long long v = v0 + u * 128;
            if (v < v_hi) {
              const long long f = flat0 + v;                         // 16-byte vector index in the flat space
              const int r = (int)(f / shard_vecs);
              buf[u] = ld_relaxed_sys_v4(reinterpret_cast<const uint4*>(p.peer_a[r]) + (f - (long long)r * shard_vecs));
            }
          }
#pragma unroll
          for (int u = 0; u < 8; ++u)
            if (v0 + u * 128 < v_hi) to[v0 + u * 128] = buf[u];
        }
        __threadfence();
        asm volatile("bar.sync 4, 128;" ::: "memory");
        if (ct == 0) {
          fence_async_proxy();
          if (atomicAdd(p.wg_cnt + blk, 1) == p.wg_parts - 1) {       // the last part of this block
            __threadfence();
            p.wg_cnt[blk] = 0;
            st_release_gpu(p.ready + blk, p.epoch);
          }
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int quarter = warp & 3;
    uint32_t local_tile = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      int b, tm, tn;
      tile_coords(tile, p, b, tm, tn);
      const int acc = local_tile & 1;
      const uint32_t acc_ph = (local_tile >> 1) & 1;
      // One lane waits, the warp follows its verdict: the tcgen05.ld below is warp-collective, so the
      // decision to go on must be uniform across the warp.
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(&acc_full[acc], acc_ph, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const int row = tm * BM + quarter * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + acc * BN + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      long long row_off = (long long)b * p.c_batch + (long long)row * p.ldc;
      void* cbase = p.C;
      if constexpr (MODE == EPI_RS) {
        // the rows of this tile belong to rank `owner`: store into its slot [self_rank][row - owner * rows_per_rank]
        const int owner = min(row / p.rows_per_rank, p.tp - 1);
        cbase = p.peer_c[owner];
        row_off = ((long long)p.self_rank * p.rows_per_rank + (row - owner * p.rows_per_rank)) * p.ldc;
      }
      if constexpr (MODE == EPI_RS) {
        // Peer stores want long contiguous pieces: transpose each 32-row x 128-column piece through this warp's
        // staging area (16-byte chunks XOR-swizzled by row) and write 256 bytes of one row per half-warp.
        uint8_t* stg = bar_base + L::BAR_BYTES + quarter * (32 * 256);
        const int row_base = tm * BM + quarter * 32;
        const int owner = min(row_base / p.rows_per_rank, p.tp - 1);
        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.peer_c[owner]) +
                             ((long long)p.self_rank * p.rows_per_rank + (row_base - owner * p.rows_per_rank)) * p.ldc;
#pragma unroll 1
        for (int hc = 0; hc < BN; hc += 128) {
#pragma unroll 1
          for (int c = 0; c < 128; c += 32) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + hc + c, r);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int e = 0; e < 4; ++e)
                vb[e] = __floats2bfloat162_rn(__uint_as_float(r[8 * q + 2 * e]), __uint_as_float(r[8 * q + 2 * e + 1]));
              const int chunk = c / 8 + q;                                   // 16-byte chunk within the 256-byte row
              *reinterpret_cast<uint4*>(stg + lane * 256 + ((chunk ^ (lane & 15)) * 16)) = v;
            }
          }
          __syncwarp();
          const int j = lane & 15;
          const int col = n0 + hc + j * 8;
#pragma unroll 4
          for (int i = 0; i < 32; i += 2) {
            const int rr = i + (lane >> 4);
            const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 256 + ((j ^ (rr & 15)) * 16));
            if (col < p.N && row_base + rr < p.M) *reinterpret_cast<uint4*>(dst + (long long)rr * p.ldc + col) = v;
          }
          __syncwarp();
        }
      } else if constexpr (MODE == EPI_CE_PARTIAL) {
        constexpr float LOG2E = 1.4426950408889634f;
        float mx = -3.0e38f;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j)
            if (n0 + c + j < p.N) mx = fmaxf(mx, __uint_as_float(r[j]));
        }
        const int y = row_ok ? (p.targets[row] - p.col0) : -1;
        float sum = 0.f, tgt = 0.f;
        const float mneg = -mx * LOG2E;
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float v = __uint_as_float(r[j]);
            if (n0 + c + j < p.N) sum += exp2f(fmaf(v, LOG2E, mneg));
            if (n0 + c + j == y) tgt = v;
          }
        }
        if (row_ok) {
          p.part[(long long)tn * p.part_stride + row] = make_float2(mx, sum);
          if (y >= n0 && y < n0 + BN && y < p.N) p.tgt_logit[row] = tgt;
        }
      } else {
      float coef = 0.f, lse = 0.f;
      int y = -1;
      if constexpr (MODE == EPI_CE_DLOGITS) {
        if (row_ok) { coef = p.row_coef[row]; lse = p.row_lse[row]; y = p.targets[row] - p.col0; }
      }
      auto xform = [&](float acc_v, int colj) -> float {
        if constexpr (MODE == EPI_CE_DLOGITS) return coef * (__expf(acc_v - lse) - (colj == y ? 1.f : 0.f));
        else return acc_v * p.alpha;
      };
      // stores and reductions as whole 128-byte lines (warp-uniform conditions; ragged column edges, odd strides and bf16
      // accumulation take the per-lane path below): the warp's piece goes through its staging area so that eight lanes
      // cover one row's 128 bytes and an instruction four rows, instead of 32 lanes touching 16 bytes of 32 rows
      const bool lines16 = !p.per_lane_stores && !p.c_is_f32 && !p.accumulate && (p.ldc & 7) == 0 &&
                           ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_batch * 2)) & 15) == 0;
      const bool lines32 = !p.per_lane_stores && p.c_is_f32 && (p.ldc & 3) == 0 &&
                           ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_batch * 4)) & 15) == 0;
      uint8_t* stg = bar_base + L::BAR_BYTES + quarter * (32 * 256);
      const int row0 = tm * BM + quarter * 32;
      const long long tile_off = (long long)b * p.c_batch + (long long)row0 * p.ldc + n0;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        if (lines16 && (c & 32) == 0 && n0 + c + 64 <= p.N) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c, r0);
          tmem_ld_32x32(taddr + c + 32, r1);
          tmem_ld_wait();
          const int col0 = n0 + c;
          stage_put_bf16x32(stg, lane, 0, r0, [&](float v, int j) { return xform(v, col0 + j); });
          stage_put_bf16x32(stg, lane, 1, r1, [&](float v, int j) { return xform(v, col0 + 32 + j); });
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
          const int col0 = n0 + c;
          stage_put_f32x32(stg, lane, r0, [&](float v, int j) { return xform(v, col0 + j); });
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
            float* out = reinterpret_cast<float*>(cbase) + row_off + col;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 v = make_float4(xform(__uint_as_float(r[j]), col + j), xform(__uint_as_float(r[j + 1]), col + j + 1),
                                       xform(__uint_as_float(r[j + 2]), col + j + 2), xform(__uint_as_float(r[j + 3]), col + j + 3));
                // C += tile: a vector reduction performed at L2 instead of load - add - store (nothing waits for a load; each
                // element is touched by one thread of one tile in a launch, so the result is the same sum)
                if (p.accumulate) red_add_f32x4(out + j, v);
                else *reinterpret_cast<float4*>(out + j) = v;
              }
            } else {
              for (int j = 0; j < 32 && col + j < p.N; ++j) {
                float v = xform(__uint_as_float(r[j]), col + j);
                if (p.accumulate) v += out[j];
                out[j] = v;
              }
            }
          } else {
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(cbase) + row_off + col;
            if (full_chunk && ((reinterpret_cast<uintptr_t>(out) & 15) == 0)) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float f[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) f[q] = xform(__uint_as_float(r[j + q]), col + j + q);
                if (p.accumulate) {
                  uint4 o = *reinterpret_cast<uint4*>(out + j);
                  const __nv_bfloat162* ob = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
                  for (int q = 0; q < 4; ++q) {
                    float2 of = __bfloat1622float2(ob[q]);
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
                float v = xform(__uint_as_float(r[j]), col + j);
                if (p.accumulate) v += __bfloat162float(out[j]);
                out[j] = __float2bfloat16(v);
              }
            }
          }
        }
      }
      }
      tc_fence_before();
      mbar_arrive(&acc_empty[acc]);
    }
    if constexpr (MODE == EPI_RS) {
      // every partial tile of this CTA is on its way to its owner: order the stores at system scope, count the CTA,
      // and let the last one raise this rank's "partials have landed" flag at every peer
      __threadfence_system();
      asm volatile("bar.sync 5, 128;" ::: "memory");
      if (threadIdx.x == 64 && ok) {
        const int prev = atomicAdd(p.done_counter, 1);
        if (prev + 1 == p.done_target) {
          __threadfence_system();
          for (int r = 0; r < p.tp; ++r) st_release_sys(p.peer_flags[r] + p.tp + p.self_rank, p.epoch);
        }
      }
    }
  }

  // ---------------------------------------------------------------- common exit
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ 256 x 256 tiles
// The same GEMM with TWO 128-row halves per tile that share every B tile: one stage holds A (2 x 16 KB) and B (32 KB), the issuer
// feeds both accumulators (TMEM columns [0, 256) and [256, 512)) from it, so a CTA pulls 64 bytes per tensor-pipe cycle from L2
// instead of 96 and three stages cover 3072 cycles of load latency instead of 2048.  The price: the accumulators are not
// double-buffered across tiles (all 512 columns belong to the current tile), so the epilogue (eight warps) is exposed; the
// launcher uses this form where the tiles are many and K is long (weight gradients over all tokens, down projections).
// Plain store epilogue only.
struct Smem256 {
  static constexpr int A_BYTES = 2 * BM * BK * 2;
  static constexpr int B_BYTES = 256 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = 3;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + 1024 + 8 * 4096 + 1024;   // stages, barriers, epilogue staging (8 warps), slack
};

__global__ void __launch_bounds__(320, 1)
gemm256_bf16_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, const GemmParams p) {
  using L = Smem256;
  constexpr int BN = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* bar_base = smem + L::STAGES * L::STAGE_BYTES;
  uint64_t* full = reinterpret_cast<uint64_t*>(bar_base);
  uint64_t* empty = full + L::STAGES;
  uint64_t* acc_full = empty + L::STAGES;
  uint64_t* acc_empty = acc_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.batch * p.tiles_m * p.tiles_n;
  const int kblocks = (p.K + BK - 1) / BK;
  constexpr uint32_t TMEM_COLS = 512;

  if (threadIdx.x == 0) {
    for (int s = 0; s < L::STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    mbar_init(acc_full, 1);
    mbar_init(acc_empty, 256);
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapA);
    tma_prefetch_desc(&mapB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int b, tm, tn;
        tile_coords(tile, p, b, tm, tn);
        const int m0 = tm * 2 * BM, n0 = tn * BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t ph = (it / L::STAGES) & 1;
          if (!mbar_wait_bounded(&empty[s], ph ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) { ok = false; break; }
          uint8_t* sA = smem + s * L::STAGE_BYTES;
          uint8_t* sB = sA + L::A_BYTES;
          mbar_expect_tx(&full[s], L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn_major) {
            tma_load_3d(sA, &mapA, &full[s], k0, m0, b);                       // box {64 k, 128 rows}, once per half
            tma_load_3d(sA + BM * BK * 2, &mapA, &full[s], k0, m0 + BM, b);
          } else {
#pragma unroll
            for (int j = 0; j < 2 * BM / 64; ++j)                              // box {64 m, 64 k-rows}
              tma_load_3d(sA + j * (BK * 128), &mapA, &full[s], m0 + j * 64, k0, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d(sB, &mapB, &full[s], k0, n0, b);                       // box {64 k, 256 rows}
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j)
              tma_load_3d(sB + j * (BK * 128), &mapB, &full[s], n0 + j * 64, k0, b);
          }
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (elect_one()) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, p.a_mn_major, p.b_mn_major);
      const uint32_t a_lbo = p.a_mn_major ? BK * 128 : 16, b_lbo = p.b_mn_major ? BK * 128 : 16;
      const uint32_t a_kstep = p.a_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t b_kstep = p.b_mn_major ? UMMA_K * 128 : UMMA_K * 2;
      const uint32_t a_half = p.a_mn_major ? 2 * (BK * 128) : BM * BK * 2;      // bytes between the two 128-row halves of A
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        if (!mbar_wait_bounded(acc_empty, (local_tile & 1) ^ 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % L::STAGES;
          const uint32_t ph = (it / L::STAGES) & 1;
          if (!mbar_wait_bounded(&full[s], ph, abort_word, p.status, ERR_WAIT_FULL)) { ok = false; break; }
          tc_fence_after();
          const uint32_t sA = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sB = sA + L::A_BYTES;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t bd = make_smem_desc(sB + k * b_kstep, b_lbo, 1024);
            umma_f16(tmem_base, make_smem_desc(sA + k * a_kstep, a_lbo, 1024), bd, idesc, (kb | k) ? 1u : 0u);
            umma_f16(tmem_base + BN, make_smem_desc(sA + a_half + k * a_kstep, a_lbo, 1024), bd, idesc, (kb | k) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        if (ok) umma_commit(acc_full);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..9: half = (warp - 2) / 4)
    const int quarter = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t local_tile = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x, ++local_tile) {
      int b, tm, tn;
      tile_coords(tile, p, b, tm, tn);
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(acc_full, local_tile & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) break;
      tc_fence_after();
      const int row = tm * 2 * BM + half * BM + quarter * 32 + lane;
      const int n0 = tn * BN;
      const uint32_t taddr = tmem_base + half * BN + ((uint32_t)(quarter * 32) << 16);
      const bool row_ok = row < p.M;
      const long long row_off = (long long)b * p.c_batch + (long long)row * p.ldc;
      // whole-line stores and reductions through a staging area, as in the 128-row kernel's epilogue
      const bool lines16 = !p.per_lane_stores && !p.c_is_f32 && !p.accumulate && (p.ldc & 7) == 0 &&
                           ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_batch * 2)) & 15) == 0;
      const bool lines32 = !p.per_lane_stores && p.c_is_f32 && (p.ldc & 3) == 0 &&
                           ((reinterpret_cast<uintptr_t>(p.C) | (uintptr_t)(p.c_batch * 4)) & 15) == 0;
      uint8_t* stg = bar_base + 1024 + (warp - 2) * 4096;
      const int row0 = tm * 2 * BM + half * BM + quarter * 32;
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
                if (p.accumulate) red_add_f32x4(out + j, v);       // see the 128-row kernel's epilogue
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
      mbar_arrive(acc_empty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 3-D bf16 tensor map {inner, outer, batch} with a 128B-swizzled box {64, box_outer, 1}.
static int make_map(CUtensorMap* map, const void* ptr, long long inner, long long outer, long long batch,
                    long long outer_stride_elems, long long batch_stride_elems, int box_outer) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return -1;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)outer, (cuuint64_t)batch};
  cuuint64_t strides[2] = {(cuuint64_t)outer_stride_elems * 2, (cuuint64_t)(batch > 1 ? batch_stride_elems : outer_stride_elems * outer) * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_outer, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  if (int c = check_map(ptr, 3, dims, strides, 2)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

// Per-device launch state: a kernel's shared-memory attribute and the SM count belong to a device, and one process may
// drive several (a C host without one-process-per-GPU).  Guarded by a mutex; indexed by the CUDA device ordinal.
constexpr int kMaxDevices = 64;
struct DeviceState {
  int num_sms = 0;
  unsigned long long attr_mask = 0;        // bit i: kernel form i has its dynamic shared-memory attribute set on this device
};
static DeviceState g_dev[kMaxDevices];
static std::mutex g_dev_mutex;

static int current_device() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

static int num_sms() {
  const int dev = current_device();
  if (dev < 0) return 148;
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (g_dev[dev].num_sms == 0) cudaDeviceGetAttribute(&g_dev[dev].num_sms, cudaDevAttrMultiProcessorCount, dev);
  return g_dev[dev].num_sms > 0 ? g_dev[dev].num_sms : 148;
}

// Run `set` once per (device, kernel form).
template <class F>
static void once_per_device(int form, F set) {
  const int dev = current_device();
  if (dev < 0) { set(); return; }
  std::lock_guard<std::mutex> lock(g_dev_mutex);
  if (!(g_dev[dev].attr_mask >> form & 1ull)) { set(); g_dev[dev].attr_mask |= 1ull << form; }
}

// The tensor-map encoder is a driver call and needs a current context in the calling thread.  Autograd runs backward
// passes on its own threads, where no runtime call may have bound the primary context yet: bind it once per thread and
// device.  `may_allocate = false` (the allocation-free entry point) binds with cudaSetDevice alone, which initialises the
// primary context since CUDA 12 without touching the allocator.
static int bind_thread_context(bool may_allocate = true) {
  static thread_local int bound_dev = -1;
  const int dev = current_device();
  if (dev < 0) return -1;
  if (bound_dev != dev) {
    if (cudaSetDevice(dev) != cudaSuccess) return -1;
    if (may_allocate) cudaFree(0);
    bound_dev = dev;
  }
  return 0;
}

template <int BN, int MODE>
static int launch_gemm(const CUtensorMap& mapA, const CUtensorMap& mapB, const GemmParams& p, int max_ctas, cudaStream_t stream) {
  once_per_device((BN == 256 ? 0 : 8) + MODE, [] {
    cudaFuncSetAttribute(gemm_bf16_kernel<BN, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         SmemLayout<BN>::TOTAL_RS);
  });
  const int sms = num_sms();
  long long tiles = (long long)p.batch * p.tiles_m * p.tiles_n;
  int cap = (max_ctas > 0 && max_ctas < sms) ? max_ctas : sms;
  int grid = (int)(tiles < cap ? tiles : cap);
  gemm_bf16_kernel<BN, MODE><<<grid, (MODE == EPI_AG || MODE == EPI_WG) ? 320 : 192,
                               SmemLayout<BN>::TOTAL_RS, stream>>>(mapA, mapB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

static int launch_gemm256(const CUtensorMap& mapA, const CUtensorMap& mapB, const GemmParams& p, cudaStream_t stream) {
  once_per_device(16, [] { cudaFuncSetAttribute(gemm256_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem256::TOTAL); });
  const int sms = num_sms();
  long long tiles = (long long)p.batch * p.tiles_m * p.tiles_n;
  int grid = (int)(tiles < sms ? tiles : sms);
  gemm256_bf16_kernel<<<grid, 320, Smem256::TOTAL, stream>>>(mapA, mapB, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

// 256 x 256 tiles pay where the grid still fills the SMs about as well as 128 x 256 tiles do (wave quantisation) and the
// exposed epilogue is short against the main loop.  DTTT_GEMM_TILE256=0 switches the form off, =1 forces it wherever it is legal.
static int g_tile256_mode = -2;            // -2: read the environment on first use; -1: automatic; 0: off; 1: wherever legal
static bool use_256_rows(int M, int N, int K, int batch, int max_ctas) {
  if (g_tile256_mode == -2) {
    const char* e = getenv("DTTT_GEMM_TILE256");
    g_tile256_mode = e ? atoi(e) : -1;
  }
  const int mode = g_tile256_mode;
  if (mode == 0 || max_ctas > 0) return false;
  if (mode == 1) return true;
  if (K < 8192) return false;               // measured: +2 % at K = 8192, +12 % at K = 49152, -6 % at K = 2048 (the exposed epilogue)
  const long long sms = num_sms();
  auto eff = [&](long long tiles) { return (double)tiles / (double)(((tiles + sms - 1) / sms) * sms); };
  const long long tn = (N + 255) / 256;
  const long long t128 = (long long)batch * ((M + 127) / 128) * tn, t256 = (long long)batch * ((M + 255) / 256) * tn;
  return eff(t256) * 1.12 >= eff(t128);
}

// Combine the per-tile (max, sum exp) partials of EPI_CE_PARTIAL into lse[row] and nll[row] = lse - target logit.
__global__ void ce_combine_kernel(const float2* __restrict__ part, long long part_stride, int tiles_n, int M,
                                  const float* __restrict__ tgt_logit, float* __restrict__ lse, float* __restrict__ nll) {
  // block = 32 rows x 8 tile-lanes; lane x owns a row, the 8 y-lanes split the column tiles
  __shared__ float sm[8][32], ss[8][32];
  const int row = blockIdx.x * 32 + threadIdx.x;
  float m = -3.0e38f, s = 0.f;
  if (row < M) {
    for (int t = threadIdx.y; t < tiles_n; t += 8) {
      const float2 v = part[(long long)t * part_stride + row];
      const float nm = fmaxf(m, v.x);
      s = s * __expf(m - nm) + v.y * __expf(v.x - nm);
      m = nm;
    }
  }
  sm[threadIdx.y][threadIdx.x] = m;
  ss[threadIdx.y][threadIdx.x] = s;
  __syncthreads();
  if (threadIdx.y == 0 && row < M) {
    float M2 = sm[0][threadIdx.x];
    for (int k = 1; k < 8; ++k) M2 = fmaxf(M2, sm[k][threadIdx.x]);
    float S2 = 0.f;
    for (int k = 0; k < 8; ++k) S2 += ss[k][threadIdx.x] * __expf(sm[k][threadIdx.x] - M2);
    const float l = M2 + logf(S2);
    lse[row] = l;
    if (nll) nll[row] = l - tgt_logit[row];
  }
}

}  // namespace dttt

using namespace dttt;

// Tile form of dttt_gemm_bf16 for N > 128: -1 automatic (the default), 0 always 128 x 256, 1 256 x 256 wherever legal.
extern "C" void dttt_gemm_tile256(int mode) { g_tile256_mode = mode; }

// C[b] (+)= alpha * A[b] x B[b].
//   a_mn_major = 0: A stored [M, K] (row stride lda);  1: A stored [K, M] (row stride lda).
//   b_mn_major = 0: B stored [N, K] (row stride ldb);  1: B stored [K, N] (row stride ldb).
// Strides are in elements; every row stride and base pointer must be a multiple of 16 bytes.
// `status` is a device int (0 = fine; see ptx_sm100.cuh for the codes).  Returns 0 on a clean launch.
extern "C" int dttt_gemm_bf16(const void* A, const void* B, void* C, int M, int N, int K, int batch,
                              long long lda, long long ldb, long long ldc, long long a_batch, long long b_batch,
                              long long c_batch, int a_mn_major, int b_mn_major, int c_is_f32, int accumulate,
                              float alpha, int* status, int max_ctas, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0 || batch <= 0) return 0;
  if ((lda % 8) || (ldb % 8) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15) ||
      (a_batch % 8) || (b_batch % 8))
    return -2;
  bind_thread_context();
  int bn = (N > 128) ? 256 : 128;
  if (bn == 256 && !use_256_rows(M, N, K, batch, max_ctas)) {
    // Small grids: 128-wide tiles when they fill the SMs so much better that the waves they need (at about 0.55 of a 256-wide
    // tile's time each) come to less than 0.85 of the 256-wide waves.  E.g. 2048 x 512: 32 tiles on 148 SMs become 64.
    const int sms = num_sms();
    const int cap = (max_ctas > 0 && max_ctas < sms) ? max_ctas : sms;
    const long long tm = (M + BM - 1) / BM;
    const long long t256 = tm * ((N + 255) / 256) * batch, t128 = tm * ((N + 127) / 128) * batch;
    const long long w256 = (t256 + cap - 1) / cap, w128 = (t128 + cap - 1) / cap;
    if (w256 <= 4 && 0.55 * (double)w128 < 0.85 * (double)w256) bn = 128;
  }
  CUtensorMap mapA, mapB;
  int r;
  if (!a_mn_major) r = make_map(&mapA, A, K, M, batch, lda, a_batch, BM);
  else             r = make_map(&mapA, A, M, K, batch, lda, a_batch, BK);
  if (r) return 100 + r;
  if (!b_mn_major) r = make_map(&mapB, B, K, N, batch, ldb, b_batch, bn);
  else             r = make_map(&mapB, B, N, K, batch, ldb, b_batch, BK);
  if (r) return 200 + r;

  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.batch = batch;
  p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.ldc = ldc; p.c_batch = c_batch; p.c_is_f32 = c_is_f32; p.accumulate = accumulate; p.alpha = alpha;
  { static const int per_lane = (getenv("DTTT_GEMM_LINES") && atoi(getenv("DTTT_GEMM_LINES")) == 0) ? 1 : 0; p.per_lane_stores = per_lane; }
  p.C = C; p.status = status;
  p.tiles_m = (M + BM - 1) / BM;
  p.tiles_n = (N + bn - 1) / bn;
  if (bn == 256 && use_256_rows(M, N, K, batch, max_ctas)) {
    p.tiles_m = (M + 2 * BM - 1) / (2 * BM);
    return launch_gemm256(mapA, mapB, p, stream);
  }
  if (bn == 256) return launch_gemm<256, EPI_STORE>(mapA, mapB, p, max_ctas, stream);
  return launch_gemm<128, EPI_STORE>(mapA, mapB, p, max_ctas, stream);
}

// Number of float2 scratch entries dttt_linear_ce_fwd needs for `rows` rows and `classes` classes.
extern "C" long long dttt_linear_ce_scratch_elems(int rows, int classes) {
  const long long stride = ((long long)rows + 127) / 128 * 128;
  return stride * ((classes + 255) / 256);
}

// Shared by the entry points that differ only in where the scratch comes from.  `may_allocate = false`: the calling
// thread's context is bound without any allocator call (the allocation-free entry point).
int dttt_linear_ce_fwd_impl(const void* h, const void* E, const int* targets, int rows, int classes, int K, long long ldh,
                            long long ldE, void* scratch, float* tgt_logit, float* lse, float* nll, int* status,
                            cudaStream_t stream, bool may_allocate = true) {
  if (rows <= 0 || classes <= 0 || K <= 0) return 0;
  if ((ldh % 8) || (ldE % 8) || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(E) & 15)) return -2;
  if (bind_thread_context(may_allocate)) return -3;
  CUtensorMap mapA, mapB;
  int r;
  if ((r = make_map(&mapA, h, K, rows, 1, ldh, 0, BM))) return 100 + r;
  if ((r = make_map(&mapB, E, K, classes, 1, ldE, 0, 256))) return 200 + r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = rows; p.N = classes; p.K = K; p.batch = 1; p.alpha = 1.f; p.status = status;
  p.tiles_m = (rows + BM - 1) / BM;
  p.tiles_n = (classes + 255) / 256;
  p.targets = targets; p.part = reinterpret_cast<float2*>(scratch); p.tgt_logit = tgt_logit;
  p.part_stride = (long long)p.tiles_m * BM;
  r = launch_gemm<256, EPI_CE_PARTIAL>(mapA, mapB, p, 0, stream);
  if (r) return r;
  ce_combine_kernel<<<(rows + 31) / 32, dim3(32, 8), 0, stream>>>(p.part, p.part_stride, p.tiles_n, rows, tgt_logit, lse, nll);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 2000 + (int)e;
}

// Forward of linear + cross-entropy: lse[r] = logsumexp_v(h_r . E_v), nll[r] = lse[r] - h_r . E_{target_r}.
//   h [rows, K] bf16 (row stride ldh), E [classes, K] bf16 (row stride ldE), targets [rows] int32.
//   scratch: dttt_linear_ce_scratch_elems(rows, classes) float2 entries of device memory (contents ignored);
//   tgt_logit, lse, nll: [rows] f32 outputs (nll may be null).  Targets outside [0, classes) leave tgt_logit untouched.
extern "C" int dttt_linear_ce_fwd(const void* h, const void* E, const int* targets, int rows, int classes, int K, long long ldh,
                                  long long ldE, void* scratch, float* tgt_logit, float* lse, float* nll, int* status,
                                  cudaStream_t stream) {
  return dttt_linear_ce_fwd_impl(h, E, targets, rows, classes, K, ldh, ldE, scratch, tgt_logit, lse, nll, status, stream);
}

// d loss / d logits for the classes [col0, col0 + ncols): D[r, c] = coef[r] * (exp(h_r . E_{col0 + c} - lse[r]) - [col0 + c == target_r])
// in bf16, row stride ldd.  Eb points at row col0 of E.
extern "C" int dttt_linear_ce_dlogits(const void* h, const void* Eb, const int* targets, const float* coef, const float* lse,
                                      void* D, int rows, int ncols, int K, long long ldh, long long ldE, long long ldd, int col0,
                                      int* status, cudaStream_t stream) {
  if (rows <= 0 || ncols <= 0 || K <= 0) return 0;
  if ((ldh % 8) || (ldE % 8) || (reinterpret_cast<uintptr_t>(h) & 15) || (reinterpret_cast<uintptr_t>(Eb) & 15)) return -2;
  bind_thread_context();
  CUtensorMap mapA, mapB;
  int r;
  if ((r = make_map(&mapA, h, K, rows, 1, ldh, 0, BM))) return 100 + r;
  if ((r = make_map(&mapB, Eb, K, ncols, 1, ldE, 0, 256))) return 200 + r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = rows; p.N = ncols; p.K = K; p.batch = 1; p.alpha = 1.f; p.status = status;
  p.ldc = ldd; p.C = D; p.c_is_f32 = 0;
  p.tiles_m = (rows + BM - 1) / BM;
  p.tiles_n = (ncols + 255) / 256;
  p.targets = targets; p.row_coef = coef; p.row_lse = lse; p.col0 = col0;
  return launch_gemm<256, EPI_CE_DLOGITS>(mapA, mapB, p, 0, stream);
}

// ------------------------------------------------------------------------------------------------------------------
// Tensor-parallel products with their collective inside the kernel (EPI_AG / EPI_RS above).

namespace dttt {
// out[i] = residual[i] + sum_s slot[s][i]: the reduction half of the fused GEMM -> reduce-scatter.  Each block first
// waits (bounded) until every rank's "partials have landed" flag has reached this epoch.
__global__ void tp_slot_reduce_kernel(const __nv_bfloat16* __restrict__ slots, const int* __restrict__ flags, int tp, int epoch,
                                      long long n_per_slot, const __nv_bfloat16* __restrict__ residual,
                                      __nv_bfloat16* __restrict__ out, int* status) {
  __shared__ int s_ok;
  __shared__ int s_abort;
  if (threadIdx.x == 0) {
    s_abort = 0;
    int ok = 1;
    for (int r = 0; r < tp && ok; ++r) ok = wait_flag_ge<true>(flags + r, epoch, &s_abort, status, ERR_WAIT_PEER) ? 1 : 0;
    s_ok = ok;
  }
  __syncthreads();
  if (!s_ok) return;
  const long long n8 = n_per_slot / 8;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float acc[8];
    if (residual) {
      const uint4 rv = reinterpret_cast<const uint4*>(residual)[i];
      const __nv_bfloat162* rb = reinterpret_cast<const __nv_bfloat162*>(&rv);
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(rb[q]); acc[2 * q] = f.x; acc[2 * q + 1] = f.y; }
    } else {
#pragma unroll
      for (int q = 0; q < 8; ++q) acc[q] = 0.f;
    }
    for (int s = 0; s < tp; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(slots + (long long)s * n_per_slot)[i];
      const __nv_bfloat162* vb = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int q = 0; q < 4; ++q) { const float2 f = __bfloat1622float2(vb[q]); acc[2 * q] += f.x; acc[2 * q + 1] += f.y; }
    }
    uint4 o;
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) ob[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

static std::mutex g_done_mutex;
static std::unordered_map<const void*, int> g_done_count;      // per counter word: CTAs counted so far
}  // namespace dttt

// C = [A_0; A_1; ...; A_{tp-1}] x B where rank r's rows live in rank r's gather buffer at the same offset.
//   peer_a[r]      rank r's gather buffer [M, K] bf16, row stride lda (elements); rank `self` has already written its
//                  own rows [self * M / tp, (self + 1) * M / tp) into peer_a[self] on this stream
//   peer_flags[r]  rank r's flag words (2 * tp ints, zero at allocation); ready: local [M / 128] ints (zero at allocation)
//   epoch          a number that grows by one per call on this set of buffers, the same on every rank
// On return (stream order) peer_a[self] holds all M rows.  M must be a multiple of 128 * tp.
extern "C" int dttt_gemm_ag_bf16(void* const* peer_a, int* const* peer_flags, int* ready, const void* B, void* C, int M, int N, int K,
                                 long long lda, long long ldb, long long ldc, int b_mn_major, int c_is_f32, int tp, int self,
                                 int epoch, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tp < 1 || tp > DTTT_MAX_TP || M % (BM * tp) || (K % 8) || (lda % 8) || (ldb % 8)) return -2;
  const void* A = peer_a[self];
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15)) return -2;
  bind_thread_context();
  const int bn = 256;
  CUtensorMap mapA, mapB;
  int r;
  if ((r = make_map(&mapA, A, K, M, 1, lda, 0, BM))) return 100 + r;
  if (!b_mn_major) r = make_map(&mapB, B, K, N, 1, ldb, 0, bn);
  else             r = make_map(&mapB, B, N, K, 1, ldb, 0, BK);
  if (r) return 200 + r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.batch = 1; p.b_mn_major = b_mn_major;
  p.ldc = ldc; p.c_is_f32 = c_is_f32; p.alpha = 1.f; p.C = C; p.status = status;
  p.tiles_m = M / BM; p.tiles_n = (N + bn - 1) / bn;
  p.tp = tp; p.self_rank = self; p.epoch = epoch; p.rows_per_rank = M / tp;
  p.m_rotate = self * (p.rows_per_rank / BM);
  p.a_row_bytes = (long long)K * 2; p.lda_bytes = lda * 2; p.ready = ready;
  for (int i = 0; i < tp; ++i) {
    if (int c = check_extent(peer_a[i], (unsigned long long)(M - 1) * lda * 2 + (unsigned long long)K * 2)) return c;
    if (int c = check_extent(peer_flags[i], (unsigned long long)2 * tp * 4)) return c;
    p.peer_a[i] = peer_a[i]; p.peer_flags[i] = peer_flags[i];
  }
  return launch_gemm<256, EPI_AG>(mapA, mapB, p, 0, stream);
}

// The host-side range check of host_check.h, whatever DTTT_DEBUG says: 0 if [ptr, ptr + bytes) lies inside one device
// allocation (or its range cannot be queried), -70 if it does not.  Nothing is launched.
extern "C" int dttt_debug_extent_check(const void* ptr, long long bytes) {
  return dttt::extent_inside_allocation(ptr, (unsigned long long)bytes);
}

// C = A x W^T (`on_k` = 0: W [N, K], rows = output columns) or C = A x W (`on_k` = 1: W [K, N], rows = contraction index) where
// the weight W is gathered inside the kernel from the ranks' flat parameter shards.
//   peer_shards[r]  rank r's shard of the flat bf16 parameter space (`shard_elems` elements; entry `self` is local)
//   flat_off        flat index of W's first element (a multiple of 8); W is dense, `w_rows` rows of `w_cols` elements
//   w_dst           local dense buffer [w_rows, w_cols] bf16 that receives the whole weight (valid after the call, stream order)
//   ready           local ints, one per 64 weight rows, zero at allocation; epoch grows by one per call on these words
//   cnt             local ints, as many, zero at allocation (how many CTAs have finished their part of a block; back to zero on exit)
// The shards must hold their final values on every rank before any rank launches, and must not change until all have finished.
extern "C" int dttt_gemm_wg_bf16(const void* A, void* const* peer_shards, void* w_dst, int* ready, int* cnt, void* C, int M, int N, int K,
                                 long long lda, long long ldc, int on_k, long long flat_off, long long shard_elems, int world,
                                 int self, int epoch, int c_is_f32, int accumulate, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  const int w_rows = on_k ? K : N, w_cols = on_k ? N : K;
  if (world < 1 || world > DTTT_MAX_TP || self < 0 || self >= world || (K % 8) || (N % 8) || (lda % 8) || (flat_off % 8) ||
      (shard_elems % 8) || shard_elems <= 0)
    return -2;
  if (on_k && (K % BK)) return -3;                      // a k-block is one 64-row copy block
  if (flat_off + (long long)w_rows * w_cols > shard_elems * world) return -4;
  if ((reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(w_dst) & 15)) return -2;
  bind_thread_context();
  const int bn = 256;
  CUtensorMap mapA, mapB;
  int r;
  if ((r = make_map(&mapA, A, K, M, 1, lda, 0, BM))) return 100 + r;
  if (!on_k) r = make_map(&mapB, w_dst, K, N, 1, K, 0, bn);
  else       r = make_map(&mapB, w_dst, N, K, 1, N, 0, BK);
  if (r) return 200 + r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.batch = 1; p.b_mn_major = on_k;
  p.ldc = ldc; p.c_is_f32 = c_is_f32; p.accumulate = accumulate; p.alpha = 1.f; p.C = C; p.status = status;
  p.tiles_m = (M + BM - 1) / BM; p.tiles_n = (N + bn - 1) / bn;
  p.tp = world; p.self_rank = self; p.epoch = epoch; p.ready = ready;
  p.wg_on_k = on_k; p.wg_rows = w_rows; p.wg_flat_off = flat_off; p.wg_shard_elems = shard_elems; p.wg_row_elems = w_cols;
  p.wg_dst = w_dst;
  // start where this rank's own part of the weight begins (if it owns any of it)
  const long long own_lo = (long long)self * shard_elems, own_hi = own_lo + shard_elems;
  const long long w_lo = flat_off, w_hi = flat_off + (long long)w_rows * w_cols;
  const long long blk_elems = (long long)WG_ROWS * w_cols;
  const int nblk = (w_rows + WG_ROWS - 1) / WG_ROWS;
  int rot = 0;
  if (own_lo < w_hi && own_hi > w_lo) rot = own_lo > w_lo ? (int)((own_lo - w_lo + blk_elems - 1) / blk_elems) : 0;
  else rot = (int)((long long)self * nblk / world);      // owns none of it: the ranks start at different blocks of the owners
  if (rot >= nblk) rot = 0;
  if (!on_k) { p.n_rotate = rot * WG_ROWS / bn; rot = p.n_rotate * (bn / WG_ROWS); }
  p.wg_rot = rot;
  // every CTA's copy warps should have something to pull: split a block's copy over several CTAs (at least 1024 vectors each)
  {
    const long long tiles = (long long)p.tiles_m * p.tiles_n;
    const int sms = num_sms();
    const int cap = (max_ctas > 0 && max_ctas < sms) ? max_ctas : sms;
    const int grid = (int)(tiles < cap ? tiles : cap);
    int parts = (grid + nblk - 1) / nblk;
    const long long vec_per_blk = blk_elems / 8;
    while (parts > 1 && vec_per_blk / parts < 1024) --parts;
    p.wg_parts = parts < 1 ? 1 : (parts > 16 ? 16 : parts);
    p.wg_cnt = cnt;
  }
  for (int i = 0; i < world; ++i) {
    if (int c = check_extent(peer_shards[i], (unsigned long long)shard_elems * 2)) return c;
    p.peer_a[i] = peer_shards[i];
  }
  if (int c = check_extent(w_dst, (unsigned long long)w_rows * w_cols * 2)) return c;
  return launch_gemm<256, EPI_WG>(mapA, mapB, p, max_ctas, stream);
}

// Partial product of this rank, reduce-scattered by rows: slot[self] of the owner of each row block receives
// alpha-free A x B tiles as they finish.  peer_c[r]: rank r's slot buffer [tp][M / tp][N] bf16; done_counter: a local
// int (zero at allocation) used only by this entry point.  Follow with dttt_tp_slot_reduce on every rank.
extern "C" int dttt_gemm_rs_bf16(const void* A, const void* B, void* const* peer_c, int* const* peer_flags, int* done_counter, int M,
                                 int N, int K, long long lda, long long ldb, int a_mn_major, int b_mn_major, int tp, int self,
                                 int epoch, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if (tp < 1 || tp > DTTT_MAX_TP || M % (BM * tp) || (N % 8) || (lda % 8) || (ldb % 8) ||
      (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -2;
  bind_thread_context();
  const int bn = (N > 128) ? 256 : 128;
  CUtensorMap mapA, mapB;
  int r;
  if (!a_mn_major) r = make_map(&mapA, A, K, M, 1, lda, 0, BM);
  else             r = make_map(&mapA, A, M, K, 1, lda, 0, BK);
  if (r) return 100 + r;
  if (!b_mn_major) r = make_map(&mapB, B, K, N, 1, ldb, 0, bn);
  else             r = make_map(&mapB, B, N, K, 1, ldb, 0, BK);
  if (r) return 200 + r;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  p.M = M; p.N = N; p.K = K; p.batch = 1; p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
  p.ldc = N; p.c_is_f32 = 0; p.alpha = 1.f; p.status = status;
  p.tiles_m = M / BM; p.tiles_n = (N + bn - 1) / bn;
  p.tp = tp; p.self_rank = self; p.epoch = epoch; p.rows_per_rank = M / tp;
  for (int i = 0; i < tp; ++i) {
    if (int c = check_extent(peer_c[i], (unsigned long long)M * N * 2)) return c;           // [tp][M / tp][N] bf16
    if (int c = check_extent(peer_flags[i], (unsigned long long)2 * tp * 4)) return c;
    p.peer_c[i] = peer_c[i]; p.peer_flags[i] = peer_flags[i];
  }
  // every rank starts with its own rows and walks the owners in ring order, so at any moment the ranks write to
  // different owners instead of all converging on one GPU's inbound links
  p.m_rotate = self * (p.rows_per_rank / BM);
  p.done_counter = done_counter;
  const long long tiles = (long long)p.tiles_m * p.tiles_n;
  const int sms = num_sms();
  const int grid = (int)(tiles < sms ? tiles : sms);
  {
    std::lock_guard<std::mutex> lock(g_done_mutex);
    p.done_target = (g_done_count[done_counter] += grid);
  }
  if (bn == 256) return launch_gemm<256, EPI_RS>(mapA, mapB, p, 0, stream);
  return launch_gemm<128, EPI_RS>(mapA, mapB, p, 0, stream);
}

// out = residual + sum over the tp slots (bf16, n_per_slot elements each, a multiple of 8); waits for every rank's flag.
extern "C" int dttt_tp_slot_reduce(const void* slots, const int* landed_flags, int tp, int epoch, long long n_per_slot,
                                   const void* residual, void* out, int* status, cudaStream_t stream) {
  if (n_per_slot <= 0) return 0;
  if (n_per_slot % 8) return -2;
  const long long n8 = n_per_slot / 8;
  const int threads = 256;
  long long blocks = (n8 + threads - 1) / threads;
  if (blocks > 148 * 8) blocks = 148 * 8;
  tp_slot_reduce_kernel<<<(int)blocks, threads, 0, stream>>>(reinterpret_cast<const __nv_bfloat16*>(slots), landed_flags, tp, epoch,
                                                            n_per_slot, reinterpret_cast<const __nv_bfloat16*>(residual),
                                                            reinterpret_cast<__nv_bfloat16*>(out), status);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}

// ------------------------------------------------------------------------------------------------------------------
// dttt_linear_ce_fwd without a caller-provided scratch buffer (see linear_ce_static.h for the contract).
#include "linear_ce_static.h"

static __device__ __align__(256) float2 g_linear_ce_scratch[DTTT_LINEAR_CE_STATIC_MAX_ELEMS];

namespace {
float2* g_scratch_addr[dttt::kMaxDevices] = {nullptr};
std::mutex g_scratch_mutex;

// Device address of the array on the current device.  The array's name is a host-side handle, not a device
// pointer: the address comes from cudaGetSymbolAddress, once per device, with that device current.
int static_scratch(float2** out) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= dttt::kMaxDevices) return DTTT_LINEAR_CE_STATIC_SETUP_FAILED;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_linear_ce_scratch) != cudaSuccess || !ptr) return DTTT_LINEAR_CE_STATIC_SETUP_FAILED;
    g_scratch_addr[dev] = reinterpret_cast<float2*>(ptr);
  }
  *out = g_scratch_addr[dev];
  return 0;
}
}  // namespace

extern "C" const char* dttt_linear_ce_static_strerror(int code) {
  switch (code) {
    case 0: return "ok";
    case DTTT_LINEAR_CE_STATIC_TOO_LARGE:
      return "dttt_linear_ce_fwd_static: ceil(rows/128)*128 * ceil(classes/256) exceeds the fixed scratch of 2097152 pairs "
             "(16 MiB); use dttt_linear_ce_fwd with a caller-allocated scratch buffer";
    case DTTT_LINEAR_CE_STATIC_SETUP_FAILED:
      return "dttt_linear_ce_fwd_static: could not resolve the device address of the scratch array on the current device";
    case -2: return "dttt_linear_ce_fwd_static: operands must be 16-byte aligned with row strides that are multiples of 8 elements";
    case -3: return "dttt_linear_ce_fwd_static: no usable current CUDA device in the calling thread";
    default: return "dttt_linear_ce_fwd_static: launch failed (tensor-map encoding or kernel launch error)";
  }
}

extern "C" int dttt_linear_ce_fwd_static(const void* h, const void* E, const int* targets, int rows, int classes, int K,
                                         long long ldh, long long ldE, float* tgt_logit, float* lse, float* nll, int* status,
                                         cudaStream_t stream) {
  if (rows <= 0 || classes <= 0 || K <= 0) return 0;
  if (dttt_linear_ce_scratch_elems(rows, classes) > DTTT_LINEAR_CE_STATIC_MAX_ELEMS) return DTTT_LINEAR_CE_STATIC_TOO_LARGE;
  float2* scratch = nullptr;
  const int r = static_scratch(&scratch);
  if (r) return r;
  // the one body both entry points run; told not to touch the allocator while binding the thread's context
  return dttt_linear_ce_fwd_impl(h, E, targets, rows, classes, K, ldh, ldE, scratch, tgt_logit, lse, nll, status, stream, false);
}
