// Chunk-window flash attention, forward, on tcgen05 tensor cores with the score and output accumulators
// in tensor memory.
//
//   O[b, i, h, :] = softmax_j( scale * Q[b, i, h, :] . K[b, j, h / rep, :] + mask(i, j) ) V[b, j, h / rep, :]
//
// Q [n, Cq, nh, d], K / V [n, Kn, nkv, d] (bf16, d contiguous), O like Q, LSE [n, nh, Cq] (f32, natural log).
// Every key is valid (the caller slices the valid suffix of the KV window, reference src/ttt/attention.py:109-120);
// `causal` aligns a causal pattern to the END of the key axis: query i sees keys j <= i + (Kn - Cq), which is the
// inner stream's own-chunk pattern with the whole window visible (reference attention.py:132-150).  GQA shares a
// K/V head among rep = nh / nkv query heads.
//
// One CTA = 128 query rows of one (sequence, head).  Per block of 128 keys:
//   warp 0     TMA: K and V tiles into a ring of shared-memory stages (128B swizzle)
//   warp 1     tcgen05.mma: S = Q K^T into one of two TMEM score buffers, then O += P V
//   warps 2-5  softmax: one thread per query row reads its score row from TMEM (tcgen05.ld), keeps the running max
//              and sum, rescales the O row in TMEM, writes P (bf16) into shared memory as the A operand of P V
// S(j+1) is issued before the softmax of block j finishes, so the tensor pipe and the exponentials overlap.
// Every wait is bounded (ptx_sm100.cuh): on a timeout the roles leave through the common exit and TMEM is freed.
#include "ptx_sm100.cuh"
#include "host_check.h"

#include <cstdlib>
#include "attn_common.cuh"

#include <mutex>
#include <cstring>

namespace dttt {

constexpr int AQ = 128;   // query rows per CTA
constexpr int AK = 128;   // keys per block

struct AttnParams {
  int n, Cq, Kn, nh, nkv, causal;
  int Kn1;              // keys [0, Kn1) come from the first K / V pair, [Kn1, Kn) from the second (Kn1 a multiple of 128, or Kn)
  float scale;
  __nv_bfloat16* O;
  float* lse;
  int* status;
  int mask_mode, mask_param;      // own-chunk pattern (two-tile kernel); `causal` is MASK_CAUSAL for the one-tile kernel
  SegSpec sg;                     // segment form (attn_common.cuh)
};

__device__ __forceinline__ SeqGeom seq_geom(const AttnParams& p, int v) {
  return seq_geom(p.sg, v, p.Cq, p.Kn, p.Kn1, p.mask_mode, p.mask_param);
}

template <int D>
struct AttnSmem {
  static constexpr int Q_BYTES = AQ * D * 2;
  static constexpr int P_BYTES = AQ * AK * 2;
  static constexpr int KV_BYTES = 2 * AK * D * 2;          // K tile + V tile
  static constexpr int STAGES = (D == 64) ? 4 : 2;
  static constexpr int TOTAL = Q_BYTES + P_BYTES + STAGES * KV_BYTES + 1024 + 1024;
};

__device__ __forceinline__ void tma_load_4d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

template <int D>
__global__ void __launch_bounds__(192, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                const __grid_constant__ CUtensorMap mapV, const AttnParams p) {
  using L = AttnSmem<D>;
  constexpr int DB = D / 64;                                // 64-wide d blocks (one 128-byte row each)
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + L::Q_BYTES;
  uint8_t* sKV = sP + L::P_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + L::STAGES * L::KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + L::STAGES;
  uint64_t* s_full = kv_empty + L::STAGES;     // [2]
  uint64_t* p_ready = s_full + 2;
  uint64_t* o_done = p_ready + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_done + 1);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.nh / p.nkv);
  const int q0 = qt * AQ;
  const int off = p.Kn - p.Cq;                              // causal alignment to the end of the key axis
  int last_key = p.Kn - 1;
  if (p.causal) last_key = min(last_key, q0 + AQ - 1 + off);
  const int nb = last_key / AK + 1;
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t S_COL0 = 0, S_COL1 = 128, O_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < L::STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
    mbar_init(p_ready, 128);
    mbar_init(o_done, 1);
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      mbar_expect_tx(q_full, L::Q_BYTES);
#pragma unroll
      for (int db = 0; db < DB; ++db) tma_load_4d(sQ + db * (AQ * 128), &mapQ, q_full, db * 64, h, q0, b);
      for (int j = 0; j < nb; ++j) {
        const int s = j % L::STAGES;
        const uint32_t ph = (j / L::STAGES) & 1;
        if (!mbar_wait_bounded(&kv_empty[s], ph ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) break;
        uint8_t* sK = sKV + s * L::KV_BYTES;
        uint8_t* sV = sK + AK * D * 2;
        mbar_expect_tx(&kv_full[s], L::KV_BYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          tma_load_4d(sK + db * (AK * 128), &mapK, &kv_full[s], db * 64, hk, j * AK, b);
          tma_load_4d(sV + db * (AK * 128), &mapV, &kv_full[s], db * 64, hk, j * AK, b);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(AQ, AK, 0, 0);          // S = Q K^T: both K-major
      const uint32_t idesc_o = make_idesc_bf16(AQ, D, 0, 1);           // O += P V: P K-major, V N-major
      const uint32_t aQ = smem_u32(sQ), aP = smem_u32(sP);
      bool ok = mbar_wait_bounded(q_full, 0, abort_word, p.status, ERR_WAIT_FULL);
      auto issue_s = [&](int j) -> bool {
        const int s = j % L::STAGES;
        if (!mbar_wait_bounded(&kv_full[s], (j / L::STAGES) & 1, abort_word, p.status, ERR_WAIT_FULL)) return false;
        tc_fence_after();
        const uint32_t aK = smem_u32(sKV + s * L::KV_BYTES);
        const uint32_t d_s = tmem + ((j & 1) ? S_COL1 : S_COL0);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t koff = (k / 4) * (AQ * 128) + (k % 4) * 32;   // 64-wide d block, then 32 bytes per UMMA_K
          umma_f16(d_s, make_smem_desc(aQ + koff, 16, 1024), make_smem_desc(aK + koff, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        umma_commit(&s_full[j & 1]);
        return true;
      };
      if (ok) ok = issue_s(0);
      for (int j = 0; j < nb && ok; ++j) {
        if (j + 1 < nb) { ok = issue_s(j + 1); if (!ok) break; }
        if (!mbar_wait_bounded(p_ready, j & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
        tc_fence_after();
        const int s = j % L::STAGES;
        const uint32_t aV = smem_u32(sKV + s * L::KV_BYTES + AK * D * 2);
#pragma unroll
        for (int k = 0; k < AK / 16; ++k) {
          const uint32_t pa = aP + (k / 4) * (AQ * 128) + (k % 4) * 32;  // P: 64-key halves, K-major
          const uint32_t va = aV + k * (16 * 128);                        // V: 16 key rows per UMMA_K
          umma_f16(tmem + O_COL, make_smem_desc(pa, 16, 1024), make_smem_desc(va, AK * 128, 1024), idesc_o, (j | k) ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(o_done);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + epilogue (one thread per row)
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;                    // row within the tile == TMEM lane
    const int qi = q0 + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const float sl2 = p.scale * 1.4426950408889634f;
    const int limit = p.causal ? (qi + off) : (p.Kn - 1);   // last visible key of this row
    float m = -1e30f, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nb; ++j) {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(&s_full[j & 1], (j >> 1) & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const uint32_t s_addr = tmem + ((j & 1) ? S_COL1 : S_COL0) + lane_addr;
      const int kbase = j * AK;
      const bool edge = (kbase + AK - 1 > limit) || (kbase + AK > p.Kn);
      // pass 1: row maximum
      float mx = m;
#pragma unroll 1
      for (int c = 0; c < AK; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float v = __uint_as_float(r[i]);
          if (edge && (kbase + c + i > limit || kbase + c + i >= p.Kn)) v = -1e30f;
          mx = fmaxf(mx, v);
        }
      }
      const float alpha = exp2f((m - mx) * sl2);
      m = mx;
      if (j > 0) {
        // P and O are free once the previous P V product has completed; then rescale this row of O
        if (lane == 0) got = mbar_wait_bounded(o_done, (j - 1) & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY) ? 1 : 0;
        got = __shfl_sync(0xffffffffu, got, 0);
        if (!got) { ok = false; break; }
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D; c += 16) {
          uint32_t r[16];
          tmem_ld_32x16(tmem + O_COL + lane_addr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x16(tmem + O_COL + lane_addr + c, r);
        }
        tmem_st_wait();
      }
      // pass 2: probabilities -> shared memory (bf16, the swizzled K-major A operand), running sum
      float sum = 0.f;
      const float mneg = -m * sl2;
#pragma unroll 1
      for (int c = 0; c < AK; c += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c, r);
        tmem_ld_wait();
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float v0 = __uint_as_float(r[i]), v1 = __uint_as_float(r[i + 1]);
          if (edge) {
            if (kbase + c + i > limit || kbase + c + i >= p.Kn) v0 = -1e30f;
            if (kbase + c + i + 1 > limit || kbase + c + i + 1 >= p.Kn) v1 = -1e30f;
          }
          const float p0 = exp2f(fmaf(v0, sl2, mneg)), p1 = exp2f(fmaf(v1, sl2, mneg));
          __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          // the sum runs over the rounded values the tensor core will see
          sum += __bfloat162float(pb.x) + __bfloat162float(pb.y);
          packed[i / 2] = *reinterpret_cast<uint32_t*>(&pb);
        }
        // 32 keys = 64 bytes = four 16-byte chunks of this row inside the 64-key half (c / 64)
        uint8_t* base = sP + (c / 64) * (AQ * 128) + (row / 8) * 1024 + (row % 8) * 128;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int chunk = (c % 64) / 8 + q;                // logical 16-byte chunk within the 128-byte row
          *reinterpret_cast<uint4*>(base + ((chunk ^ (row % 8)) * 16)) =
              make_uint4(packed[4 * q], packed[4 * q + 1], packed[4 * q + 2], packed[4 * q + 3]);
        }
      }
      l = l * alpha + sum;
      fence_async_proxy();
      tc_fence_before();
      mbar_arrive(p_ready);
    }
    if (ok) {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(o_done, (nb - 1) & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* out = p.O + (((long long)b * p.Cq + qi) * p.nh + h) * D;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(tmem + O_COL + lane_addr + c, r);
          tmem_ld_wait();
          if (qi < p.Cq) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                vb[q] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * q]) * inv, __uint_as_float(r[i + 2 * q + 1]) * inv);
              *reinterpret_cast<uint4*>(out + c + i) = v;
            }
          }
        }
        if (qi < p.Cq && p.lse) p.lse[((long long)b * p.nh + h) * p.Cq + qi] = m * p.scale + logf(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ------------------------------------------------------------------------------------------------------------------
// Second version: two 128-row query tiles per CTA in ping-pong, P kept in tensor memory.
//
//   warp 0      TMA: Q (both tiles) once, then K / V stages
//   warp 1      tcgen05.mma issuer.  Per key block and tile: O_t += P_t V (A operand read from TMEM), then the
//               next S_t = Q_t K^T into the same TMEM columns P_t occupied; the tensor pipe runs its queue in order,
//               so tile A's products run while tile B's softmax computes and the other way round
//   warps 2-5   softmax of tile A, warps 6-9 of tile B: one thread per row holds the 128 scores of the block in
//               registers, writes P (bf16 pairs) back over the first 64 columns of its S row
//   (Two threads per row on sixteen softmax warps, agreeing on the row maximum through shared memory once per block, was
//               built and measured: 1.276 against 1.085 ms at 8 x 1024 x 9216 causal with heads of 64, 0.731 against 0.649 ms
//               with heads of 128 - slower, the exchange and its barrier cost more than the extra warps hide - and taken out.)
// The running maximum is only raised when a row's block maximum exceeds it by more than 2^8 (in the exponent's
// units), so most blocks skip the read-modify-write of the O row; the final O / l and the LSE are exact either way.
// TMEM columns: S_A / P_A [0,128)  S_B / P_B [128,256)  O_A [256,256+D)  O_B [256+D,256+2D).
template <int D>
struct Attn2Smem {
  static constexpr int Q_BYTES = 2 * AQ * D * 2;
  static constexpr int KV_BYTES = 2 * AK * D * 2;
  static constexpr int STAGES = (D == 64) ? 4 : 2;
  static constexpr int TOTAL = Q_BYTES + STAGES * KV_BYTES + 1024 + 1024;
};

template <int D>
__global__ void __launch_bounds__(320, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap mapQ, const __grid_constant__ CUtensorMap mapK,
                 const __grid_constant__ CUtensorMap mapV, const __grid_constant__ CUtensorMap mapK2,
                 const __grid_constant__ CUtensorMap mapV2, const AttnParams p) {
  using L = Attn2Smem<D>;
  constexpr int DB = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sKV = sQ + L::Q_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sKV + L::STAGES * L::KV_BYTES);
  uint64_t* q_full = bars;
  uint64_t* kv_full = bars + 1;
  uint64_t* kv_empty = kv_full + L::STAGES;
  uint64_t* s_full = kv_empty + L::STAGES;     // [2] one per tile
  uint64_t* p_ready = s_full + 2;              // [2]
  uint64_t* o_final = p_ready + 2;             // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(o_final + 2);
  volatile int* abort_word = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = gridDim.x - 1 - blockIdx.x;                // longest (latest) query tiles first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hk = h / (p.nh / p.nkv);
  const SeqGeom G = seq_geom(p, b);
  // The sub-block read leaves a gap in a row's keys and the two tiles of a CTA would walk different block lists:
  // it runs one tile per CTA.  Every other pattern is a prefix of the key axis per row.
  const bool single = G.mode == MASK_READ;
  const int q0 = single ? qt * AQ : qt * 2 * AQ;
  int nb[2], n1[2];
  int gap_from = 0, gap_to = 0;                             // second block range of the single-tile form: [gap_to, ...) follows n1
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int i0 = q0 + t * AQ, i1 = min(i0 + AQ - 1, p.Cq - 1);
    nb[t] = n1[t] = 0;
    if (i0 < p.Cq && !(single && t == 1)) {
      const RowMask last = row_mask(G.mode, G.param, i1, G.Kn, p.Cq);
      n1[t] = last.e1 >= 0 ? last.e1 / AK + 1 : 0;
      nb[t] = n1[t];
      if (single) {
        const RowMask first = row_mask(G.mode, G.param, i0, G.Kn, p.Cq);
        gap_from = n1[t];
        gap_to = max(first.s2 / AK, n1[t]);
        nb[t] = n1[t] + (last.e2 / AK - gap_to + 1);
      }
    }
  }
  const int nbmax = max(nb[0], nb[1]);
  // entry jj of the block list -> key block
  auto blk = [&](int jj) { return (single && jj >= gap_from) ? gap_to + (jj - gap_from) : jj; };
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t O_COL = 256;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < L::STAGES; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int t = 0; t < 2; ++t) { mbar_init(&s_full[t], 1); mbar_init(&p_ready[t], 128); mbar_init(&o_final[t], 1); }
    *abort_word = 0;
    fence_mbar_init();
    tma_prefetch_desc(&mapQ); tma_prefetch_desc(&mapK); tma_prefetch_desc(&mapV);
    tma_prefetch_desc(&mapK2); tma_prefetch_desc(&mapV2);
  }
  if (warp == 1) { tmem_alloc(tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      mbar_expect_tx(q_full, (nb[1] > 0 ? 2 : 1) * (L::Q_BYTES / 2));
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int db = 0; db < DB; ++db)
          if (nb[t] > 0 || t == 0) tma_load_4d(sQ + t * (AQ * D * 2) + db * (AQ * 128), &mapQ, q_full, db * 64, h, q0 + t * AQ, b);
      for (int j = 0; j < nbmax; ++j) {
        const int s = j % L::STAGES;
        const uint32_t ph = (j / L::STAGES) & 1;
        if (!mbar_wait_bounded(&kv_empty[s], ph ^ 1, abort_word, p.status, ERR_WAIT_EMPTY)) break;
        uint8_t* sK = sKV + s * L::KV_BYTES;
        uint8_t* sV = sK + AK * D * 2;
        mbar_expect_tx(&kv_full[s], L::KV_BYTES);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
          // the window (first pair) and the chunk's own keys (second pair) are separate tensors: no concatenation pass
          const int k0 = blk(j) * AK;
          const bool second = k0 >= G.Kn1;
          const int krow = second ? k0 - G.Kn1 : G.row0 + k0;
          const int kbat = second ? b : G.kb;
          tma_load_4d(sK + db * (AK * 128), second ? &mapK2 : &mapK, &kv_full[s], db * 64, hk, krow, kbat);
          tma_load_4d(sV + db * (AK * 128), second ? &mapV2 : &mapV, &kv_full[s], db * 64, hk, krow, kbat);
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      const uint32_t idesc_s = make_idesc_bf16(AQ, AK, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(AQ, D, 0, 1);
      bool ok = mbar_wait_bounded(q_full, 0, abort_word, p.status, ERR_WAIT_FULL);
      int loaded = -1;                                       // newest key block whose stage is known to be full
      auto issue_s = [&](int t, int j) -> bool {
        const int s = j % L::STAGES;
        if (j > loaded) {
          if (!mbar_wait_bounded(&kv_full[s], (j / L::STAGES) & 1, abort_word, p.status, ERR_WAIT_FULL)) return false;
          tc_fence_after();
          loaded = j;
        }
        const uint32_t aQ = smem_u32(sQ + t * (AQ * D * 2));
        const uint32_t aK = smem_u32(sKV + s * L::KV_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint32_t koff = (k / 4) * (AQ * 128) + (k % 4) * 32;
          umma_f16(tmem + t * 128, make_smem_desc(aQ + koff, 16, 1024), make_smem_desc(aK + koff, 16, 1024), idesc_s, k ? 1u : 0u);
        }
        umma_commit(&s_full[t]);
        return true;
      };
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (ok && nb[t] > 0) ok = issue_s(t, 0);
      for (int j = 0; j < nbmax && ok; ++j) {
        const int s = j % L::STAGES;
        const uint32_t aV = smem_u32(sKV + s * L::KV_BYTES + AK * D * 2);
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (!ok || j >= nb[t]) continue;
          if (!mbar_wait_bounded(&p_ready[t], j & 1, abort_word, p.status, ERR_WAIT_TMEM_EMPTY)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < AK / 16; ++k)                  // 16 keys = 8 TMEM columns of packed bf16 pairs
            umma_f16_ts(tmem + O_COL + t * D, tmem + t * 128 + k * 8, make_smem_desc(aV + k * (16 * 128), AK * 128, 1024),
                        idesc_o, (j | k) ? 1u : 0u);
          if (j + 1 < nb[t]) ok = issue_s(t, j + 1);
          else umma_commit(&o_final[t]);
        }
        if (ok) umma_commit(&kv_empty[s]);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax + epilogue
    const int t = (warp - 2) >> 2;                          // tile of this warpgroup
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int qi = q0 + t * AQ + row;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_addr = tmem + t * 128 + lane_addr;
    const uint32_t o_addr = tmem + O_COL + t * D + lane_addr;
    const float sl2 = p.scale * 1.4426950408889634f;
    const RowMask rm = row_mask(G.mode, G.param, min(qi, p.Cq - 1), G.Kn, p.Cq);
    float m = -1e30f, l = 0.f;
    bool ok = true;
    const int nbt = nb[t];
    for (int j = 0; j < nbt; ++j) {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(&s_full[t], j & 1, abort_word, p.status, ERR_WAIT_TMEM_FULL) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (!got) { ok = false; break; }
      tc_fence_after();
      const int kbase = blk(j) * AK;
      const bool whole = (kbase + AK - 1 <= rm.e1) || (kbase >= rm.s2 && kbase + AK - 1 <= rm.e2);
      // columns of this block the row sees: [0, hi1] (prefix interval) and [lo2, hi2] (second interval)
      const int hi1 = rm.e1 - kbase, lo2 = rm.s2 - kbase, hi2 = rm.e2 - kbase;
      // One pass over the block: its scores from TMEM, exponentials against the reference maximum `m_ref`, the block maximum
      // tracked alongside (the two interleave; a separate maximum pass would sit in front of the first ex2), P packed.
      float sum0, sum1, mx;
      uint32_t pk[64];
      auto exp_block = [&](float m_ref) {
        uint32_t sr[128];
        tmem_ld_32x32(s_addr + 0, reinterpret_cast<uint32_t(&)[32]>(sr[0]));
        tmem_ld_32x32(s_addr + 32, reinterpret_cast<uint32_t(&)[32]>(sr[32]));
        tmem_ld_32x32(s_addr + 64, reinterpret_cast<uint32_t(&)[32]>(sr[64]));
        tmem_ld_32x32(s_addr + 96, reinterpret_cast<uint32_t(&)[32]>(sr[96]));
        tmem_ld_wait();
        if (!whole) {
#pragma unroll
          for (int i = 0; i < 128; ++i)
            if (i > hi1 && (i < lo2 || i > hi2)) sr[i] = __float_as_uint(MASKED);
        }
        const float mneg = -m_ref * sl2;
        float mx0 = -3.4e38f, mx1 = -3.4e38f, s0 = 0.f, s1 = 0.f;
#pragma unroll
        for (int i = 0; i < 128; i += 2) {
          const float a0 = __uint_as_float(sr[i]), a1 = __uint_as_float(sr[i + 1]);
          mx0 = fmaxf(mx0, a0); mx1 = fmaxf(mx1, a1);
          const float p0 = ex2_approx(fmaf(a0, sl2, mneg));
          const float p1 = ex2_approx(fmaf(a1, sl2, mneg));
          s0 += p0; s1 += p1;
          __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
          pk[i / 2] = *reinterpret_cast<uint32_t*>(&pb);
        }
        sum0 = s0; sum1 = s1; mx = fmaxf(mx0, mx1);
      };
      exp_block(m);
      // Only when the block raises the maximum by more than 2^8 in the exponent's units - rare after the first blocks - is the
      // reference raised and the block done again from its scores, which are still in TMEM (P has not been stored yet).
      // (warp-uniform decision: the TMEM accesses are collective)
      if (__any_sync(0xffffffffu, (mx - m) * sl2 > 8.f)) {
        const float m_new = fmaxf(m, mx);
        const float alpha = exp2f((m - m_new) * sl2);
        m = m_new;
        l *= alpha;
        if (j > 0) {
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32(o_addr + c, o);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32(o_addr + c, o);
          }
        }
        exp_block(m);
      }
      l += sum0 + sum1;
      tmem_st_32x32(s_addr + 0, reinterpret_cast<uint32_t(&)[32]>(pk[0]));
      tmem_st_32x32(s_addr + 32, reinterpret_cast<uint32_t(&)[32]>(pk[32]));
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_ready[t]);
    }
    if (ok && nbt > 0) {
      int got = 1;
      if (lane == 0) got = mbar_wait_bounded(&o_final[t], 0, abort_word, p.status, ERR_WAIT_TMEM_EMPTY) ? 1 : 0;
      got = __shfl_sync(0xffffffffu, got, 0);
      if (got) {
        tc_fence_after();
        const float inv = 1.f / l;
        __nv_bfloat16* out = p.O + (((long long)b * p.Cq + qi) * p.nh + h) * D;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t r[32];
          tmem_ld_32x32(o_addr + c, r);
          tmem_ld_wait();
          if (qi < p.Cq) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 v;
              __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
              for (int q = 0; q < 4; ++q)
                vb[q] = __floats2bfloat162_rn(__uint_as_float(r[i + 2 * q]) * inv, __uint_as_float(r[i + 2 * q + 1]) * inv);
              *reinterpret_cast<uint4*>(out + c + i) = v;
            }
          }
        }
        if (qi < p.Cq && p.lse) p.lse[((long long)b * p.nh + h) * p.Cq + qi] = m * p.scale + logf(l);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

typedef CUresult (*EncodeTiledFn4)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                   const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn4 attn_encode_fn() {
  static EncodeTiledFn4 fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn4>(ptr);
  });
  return fn;
}

// [n, rows, heads, d] bf16 with d contiguous; box = 64 d x 1 head x 128 rows x 1
static int make_map4(CUtensorMap* map, const void* ptr, int n, int rows, int heads, int d, long long batch_stride = 0) {
  EncodeTiledFn4 enc = attn_encode_fn();
  if (!enc) return -1;
  if (batch_stride <= 0) batch_stride = (long long)rows * heads * d;      // elements between sequences (a slice of a longer window has more)
  cuuint64_t dims[4] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)rows, (cuuint64_t)n};
  cuuint64_t strides[3] = {(cuuint64_t)d * 2, (cuuint64_t)heads * d * 2, (cuuint64_t)batch_stride * 2};
  cuuint32_t box[4] = {64, 1, 128, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  if (int c = check_map(ptr, 4, dims, strides, 2)) return c;
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

}  // namespace dttt

namespace dttt {
template <int D>
static int launch_fwd2(dim3 grid, const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const CUtensorMap& mk2,
                       const CUtensorMap& mv2, const AttnParams& p, cudaStream_t stream) {
  static bool attr = false;
  if (!attr) { cudaFuncSetAttribute(attn_fwd2_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, Attn2Smem<D>::TOTAL); attr = true; }
  attn_fwd2_kernel<D><<<grid, 320, Attn2Smem<D>::TOTAL, stream>>>(mq, mk, mv, mk2, mv2, p);
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}
}  // namespace dttt

using namespace dttt;

// Q [n, Cq, nh, d], O like Q (bf16, contiguous), lse [n, nh, Cq] f32 or null, d in {64, 128}.  Keys and values may come
// as two pairs: K / V [n, Kn1, nkv, d] followed by K2 / V2 [n, Kn2, nkv, d] (rows contiguous, `*_bs` = elements between
// sequences, so a slice of a longer window needs no copy); K2 == null means one pair of Kn1 keys.  With two pairs Kn1 must be
// a multiple of 128 and the two-tile variant (0) is used.
extern "C" int dttt_attn_fwd(const void* Q, const void* K, const void* V, const void* K2, const void* V2, void* O, float* lse, int n,
                             int Cq, int Kn1, int Kn2, int nh, int nkv, int d, long long k_bs, long long v_bs, long long k2_bs,
                             long long v2_bs, float scale, int causal, int variant, int* status, cudaStream_t stream) {
  const int Kn = Kn1 + (K2 ? Kn2 : 0);
  if ((d != 64 && d != 128) || nh % nkv || n <= 0 || Cq <= 0 || Kn <= 0) return -2;
  if (causal && Kn < Cq) return -3;
  if (K2 && (Kn1 % AK || variant != 0)) return -4;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { int dev = 0; cudaGetDevice(&dev); cudaSetDevice(dev); cudaFree(0); ctx_bound = true; }
  CUtensorMap mq, mk, mv, mk2, mv2;
  int r;
  if ((r = make_map4(&mq, Q, n, Cq, nh, d))) return 100 + r;
  if ((r = make_map4(&mk, K, n, Kn1, nkv, d, k_bs))) return 200 + r;
  if ((r = make_map4(&mv, V, n, Kn1, nkv, d, v_bs))) return 300 + r;
  if (K2) {
    if ((r = make_map4(&mk2, K2, n, Kn2, nkv, d, k2_bs))) return 400 + r;
    if ((r = make_map4(&mv2, V2, n, Kn2, nkv, d, v2_bs))) return 500 + r;
  } else {
    mk2 = mk; mv2 = mv;
  }
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.n = n; p.Cq = Cq; p.Kn = Kn; p.Kn1 = K2 ? Kn1 : Kn; p.nh = nh; p.nkv = nkv; p.causal = causal; p.scale = scale;
  p.O = reinterpret_cast<__nv_bfloat16*>(O); p.lse = lse; p.status = status;
  p.mask_mode = causal ? MASK_CAUSAL : MASK_FULL;
  if (variant == 0) {
    dim3 grid2((Cq + 2 * AQ - 1) / (2 * AQ), nh, n);
    return d == 64 ? launch_fwd2<64>(grid2, mq, mk, mv, mk2, mv2, p, stream) : launch_fwd2<128>(grid2, mq, mk, mv, mk2, mv2, p, stream);
  }
  dim3 grid((Cq + AQ - 1) / AQ, nh, n);
  static bool attr64 = false, attr128 = false;
  if (d == 64) {
    if (!attr64) { cudaFuncSetAttribute(attn_fwd_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<64>::TOTAL); attr64 = true; }
    attn_fwd_kernel<64><<<grid, 192, AttnSmem<64>::TOTAL, stream>>>(mq, mk, mv, p);
  } else {
    if (!attr128) { cudaFuncSetAttribute(attn_fwd_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<128>::TOTAL); attr128 = true; }
    attn_fwd_kernel<128><<<grid, 192, AttnSmem<128>::TOTAL, stream>>>(mq, mk, mv, p);
  }
  cudaError_t e = cudaGetLastError();
  return e == cudaSuccess ? 0 : 1000 + (int)e;
}



// The forward with an own-chunk pattern: mode 0 full, 1 causal, 2 split (param = context length), 3 block (param = sub-block),
// 4 sub-block read (param = sub-block; the keys are [window | clean own chunk | own chunk], Kn1 counts the first two).  Cq must be
// a multiple of 128 for modes 2-4.  Arguments otherwise as dttt_attn_fwd with two key / value pairs.
extern "C" int dttt_attn_fwd_masked(const void* Q, const void* K, const void* V, const void* K2, const void* V2, void* O, float* lse, int n,
                                    int Cq, int Kn1, int Kn2, int nh, int nkv, int d, long long k_bs, long long v_bs, long long k2_bs,
                                    long long v2_bs, float scale, int mode, int param, int* status, cudaStream_t stream) {
  const int Kn = Kn1 + (K2 ? Kn2 : 0);
  if ((d != 64 && d != 128) || nh % nkv || n <= 0 || Cq <= 0 || Kn < Cq || mode < 0 || mode > MASK_READ) return -2;
  if (mode >= MASK_SPLIT && (Cq % AK || param <= 0 || param > Cq)) return -3;
  if (mode == MASK_READ && Kn < 2 * Cq) return -3;
  if (K2 && Kn1 % AK) return -4;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { int dev = 0; cudaGetDevice(&dev); cudaSetDevice(dev); cudaFree(0); ctx_bound = true; }
  CUtensorMap mq, mk, mv, mk2, mv2;
  int r;
  if ((r = make_map4(&mq, Q, n, Cq, nh, d))) return 100 + r;
  if (Kn1 > 0) {
    if ((r = make_map4(&mk, K, n, Kn1, nkv, d, k_bs))) return 200 + r;
    if ((r = make_map4(&mv, V, n, Kn1, nkv, d, v_bs))) return 300 + r;
  }
  if (K2) {
    if ((r = make_map4(&mk2, K2, n, Kn2, nkv, d, k2_bs))) return 400 + r;
    if ((r = make_map4(&mv2, V2, n, Kn2, nkv, d, v2_bs))) return 500 + r;
    if (Kn1 == 0) { mk = mk2; mv = mv2; }
  } else {
    mk2 = mk; mv2 = mv;
  }
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.n = n; p.Cq = Cq; p.Kn = Kn; p.Kn1 = K2 ? Kn1 : Kn; p.nh = nh; p.nkv = nkv; p.causal = mode == MASK_CAUSAL; p.scale = scale;
  p.O = reinterpret_cast<__nv_bfloat16*>(O); p.lse = lse; p.status = status;
  p.mask_mode = mode; p.mask_param = param;
  const int tiles = mode == MASK_READ ? (Cq + AQ - 1) / AQ : (Cq + 2 * AQ - 1) / (2 * AQ);
  dim3 grid(tiles, nh, n);
  return d == 64 ? launch_fwd2<64>(grid, mq, mk, mv, mk2, mv2, p, stream) : launch_fwd2<128>(grid, mq, mk, mv, mk2, mv2, p, stream);
}

// Segment form: every chunk of every stream of a [B, streams, chunks * C] segment in ONE launch, the clean windows read in place.
//   Q, O          [B, streams, chunks * C, nh, d]   (contiguous)       lse [B * streams * chunks, nh, C]
//   Kc, Vc        the clean stream's keys / values with the window of the previous segment in front: [B, (W + chunks) * C, nkv, d],
//                 `kc_bs` / `vc_bs` elements between sequences
//   Ko, Vo        every stream's own keys / values [B, streams, chunks * C, nkv, d] (contiguous)
//   first         index within the sequence of the segment's first chunk; reach < 0: no limit on the window
//   modes, params per stream own-chunk pattern (as dttt_attn_fwd_masked; a stream in read mode finds the clean own chunk right
//                 behind its window in Kc / Vc)
extern "C" int dttt_attn_fwd_segment(const void* Q, const void* Kc, const void* Vc, const void* Ko, const void* Vo, void* O, float* lse,
                                     int B, int streams, int chunks, int C, int W, int first, int reach, int nh, int nkv, int d,
                                     long long kc_bs, long long vc_bs, const int* modes, const int* params, float scale, int* status,
                                     cudaStream_t stream) {
  if ((d != 64 && d != 128) || nh % nkv || B <= 0 || streams <= 0 || streams > MAX_STREAMS || chunks <= 0 || C % AK || W < 0) return -2;
  static thread_local bool ctx_bound = false;
  if (!ctx_bound) { int dev = 0; cudaGetDevice(&dev); cudaSetDevice(dev); cudaFree(0); ctx_bound = true; }
  const int n = B * streams * chunks;
  CUtensorMap mq, mk, mv, mk2, mv2;
  int r;
  if ((r = make_map4(&mq, Q, n, C, nh, d))) return 100 + r;
  if ((r = make_map4(&mk, Kc, B, (W + chunks) * C, nkv, d, kc_bs))) return 200 + r;
  if ((r = make_map4(&mv, Vc, B, (W + chunks) * C, nkv, d, vc_bs))) return 300 + r;
  if ((r = make_map4(&mk2, Ko, n, C, nkv, d))) return 400 + r;
  if ((r = make_map4(&mv2, Vo, n, C, nkv, d))) return 500 + r;
  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.n = n; p.Cq = C; p.nh = nh; p.nkv = nkv; p.scale = scale;
  p.O = reinterpret_cast<__nv_bfloat16*>(O); p.lse = lse; p.status = status;
  p.sg.on = 1; p.sg.streams = streams; p.sg.chunks = chunks; p.sg.first = first; p.sg.W = W; p.sg.reach = reach;
  bool any_read = false;
  for (int s = 0; s < streams; ++s) {
    p.sg.mode[s] = modes[s]; p.sg.param[s] = params[s];
    if (modes[s] < 0 || modes[s] > MASK_READ || (modes[s] >= MASK_SPLIT && (params[s] <= 0 || params[s] > C))) return -3;
    any_read |= modes[s] == MASK_READ;
  }
  // one tile per CTA when a stream uses the read pattern (its CTAs walk a block list with a gap); the others then simply run
  // their second tile as a CTA of its own
  if (any_read) return -5;
  dim3 grid((C + 2 * AQ - 1) / (2 * AQ), nh, n);
  return d == 64 ? launch_fwd2<64>(grid, mq, mk, mv, mk2, mv2, p, stream) : launch_fwd2<128>(grid, mq, mk, mv, mk2, mv2, p, stream);
}
