// Gated delta rule over one chunk in the blocked (WY / UT-transform) form, forward and backward, exact f32.
//
//   S_t = a_t S_{t-1} + b_t (v_t - a_t S_{t-1} k_t) k_t^T          S [dv, dk] per (sequence, head)
//
// (reference src/ttt/gdn.py:106-123; its plain loop :125-136 is the oracle).  Over a block of L = 64 tokens with
// g_i = sum_{j<=i} log a_j the recurrence has the closed form
//
//   A   = strict_lower( diag(b) (K K^T) .* exp(g_i - g_j) )          T = (I + A)^-1  (unit lower triangular)
//   W   = V - diag(e^g) K S0^T          R = diag(b) W          U = T R
//   S_L = e^{g_L} S0 + U^T diag(e^{g_L - g}) K
//
// so a chunk of C tokens is C / 64 block steps of small dense products instead of C rank-one updates, and the
// backward is the same block steps in reverse with the state at every block boundary re-created by a forward sweep.
//
// Rows of S evolve independently given (K, b, g): the state of a head is split into slices of RS = 32 value rows,
// one CTA per (slice, head, sequence), which fills the machine (B x heads x dv / 32 CTAs) and lets a slice of the
// state, its gradient and every block-sized operand live in shared memory.  What is shared between the slices of a
// head (dK, d beta, d log a) is written as one partial per slice and summed by the caller; dV and dS0 are owned by a
// slice.  Everything is f32 FMA arithmetic: the products are tiny (6 MFLOP per block) and the point of this kernel is
// to replace some hundred launches per chunk by one, with the exact arithmetic of the oracle.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int L = 64;        // tokens per block
constexpr int RS = 32;       // value rows of the state per CTA
constexpr int NT = 256;      // threads per CTA

// C[i*ldc + j] (+)= alpha * sum_k A[i*sai + k*sak] * B[k*sbk + j*sbj]   (i < M, j < N), whole CTA.
// kmin / kmax callbacks would complicate things; triangular products simply multiply by stored zeros.
template <bool ACC>
__device__ __forceinline__ void mm(float* C, int ldc, const float* A, int sai, int sak, const float* B, int sbk, int sbj,
                                   int M, int N, int K, float alpha = 1.f) {
  for (int idx = threadIdx.x; idx < M * N; idx += NT) {
    const int i = idx / N, j = idx - i * N;
    const float* a = A + i * sai;
    const float* b = B + j * sbj;
    float acc = 0.f;
#pragma unroll 8
    for (int k = 0; k < K; ++k) acc = fmaf(a[k * sak], b[k * sbk], acc);
    if (ACC) C[i * ldc + j] += alpha * acc;
    else C[i * ldc + j] = alpha * acc;
  }
}

template <int D>
struct Smem {
  // leading dimensions padded by one float so that column walks do not hit one bank
  static constexpr int LDK = D + 1, LDR = RS + 1, LDL = L + 1;
  float K[L * LDK];        // keys of the block
  float X[L * LDK];        // backward: dK of the block (this slice's part)
  float S[RS * LDK];       // state slice (at the start of the block)
  float G[RS * LDK];       // backward: gradient w.r.t. the state slice after the block
  float A[L * LDL];        // A, then reused
  float T[L * LDL];        // (I + A)^-1
  float M[L * LDL];        // K K^T
  float dA[L * LDL];       // backward
  float V[L * LDR], P[L * LDR], W[L * LDR], U[L * LDR], dU[L * LDR], dR[L * LDR];
  float beta[L], g[L], eg[L], dec[L], dbeta[L], dg[L];
  float red[NT / 32];
};

// Loads block n of (k, v slice, beta, log alpha), forms g / e^g / e^{gL - g}, M = K K^T, A, T, P, W, R (in dR's place
// only transiently), U.  On return sm.S still holds the block's initial state.
template <int D>
__device__ void block_forward_parts(Smem<D>& sm, const float* __restrict__ k, const float* __restrict__ v,
                                    const float* __restrict__ beta, const float* __restrict__ la, long long tok0, int nh, int h,
                                    int row0) {
  using SM = Smem<D>;
  for (int idx = threadIdx.x; idx < L * D; idx += NT) {
    const int i = idx / D, c = idx - i * D;
    sm.K[i * SM::LDK + c] = k[((tok0 + i) * nh + h) * D + c];
  }
  for (int idx = threadIdx.x; idx < L * RS; idx += NT) {
    const int i = idx / RS, r = idx - i * RS;
    sm.V[i * SM::LDR + r] = v[((tok0 + i) * nh + h) * D + row0 + r];
  }
  if (threadIdx.x < L) {
    sm.beta[threadIdx.x] = beta[(tok0 + threadIdx.x) * nh + h];
    sm.g[threadIdx.x] = la[(tok0 + threadIdx.x) * nh + h];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    float run = 0.f;
    for (int i = 0; i < L; ++i) { run += sm.g[i]; sm.g[i] = run; }
  }
  __syncthreads();
  if (threadIdx.x < L) {
    sm.eg[threadIdx.x] = __expf(sm.g[threadIdx.x]);
    sm.dec[threadIdx.x] = __expf(sm.g[L - 1] - sm.g[threadIdx.x]);
  }
  mm<false>(sm.M, SM::LDL, sm.K, SM::LDK, 1, sm.K, 1, SM::LDK, L, L, D);
  __syncthreads();
  for (int idx = threadIdx.x; idx < L * L; idx += NT) {
    const int i = idx / L, j = idx - i * L;
    sm.A[i * SM::LDL + j] = (i > j) ? sm.beta[i] * sm.M[i * SM::LDL + j] * __expf(sm.g[i] - sm.g[j]) : 0.f;
  }
  __syncthreads();
  // T = (I + A)^-1 by forward substitution, one thread per column: T[i][c] = [i == c] - sum_{j < i} A[i][j] T[j][c]
  if (threadIdx.x < L) {
    const int c = threadIdx.x;
    for (int i = 0; i < L; ++i) {
      float t = (i == c) ? 1.f : 0.f;
      for (int j = c; j < i; ++j) t = fmaf(-sm.A[i * SM::LDL + j], sm.T[j * SM::LDL + c], t);
      sm.T[i * SM::LDL + c] = (i >= c) ? t : 0.f;
    }
  }
  // P = K S^T   [L, RS]
  mm<false>(sm.P, SM::LDR, sm.K, SM::LDK, 1, sm.S, 1, SM::LDK, L, RS, D);
  __syncthreads();
  for (int idx = threadIdx.x; idx < L * RS; idx += NT) {
    const int i = idx / RS, r = idx - i * RS;
    const float w = sm.V[i * SM::LDR + r] - sm.eg[i] * sm.P[i * SM::LDR + r];
    sm.W[i * SM::LDR + r] = w;
    sm.dR[i * SM::LDR + r] = sm.beta[i] * w;          // R, transiently
  }
  __syncthreads();
  mm<false>(sm.U, SM::LDR, sm.T, SM::LDL, 1, sm.dR, SM::LDR, 1, L, RS, L);
  __syncthreads();
}

// S <- e^{gL} S + U^T diag(dec) K
template <int D>
__device__ void block_state_update(Smem<D>& sm) {
  using SM = Smem<D>;
  const float egl = sm.eg[L - 1];
  for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
    const int r = idx / D, c = idx - r * D;
    float acc = egl * sm.S[r * SM::LDK + c];
#pragma unroll 8
    for (int i = 0; i < L; ++i) acc = fmaf(sm.U[i * SM::LDR + r] * sm.dec[i], sm.K[i * SM::LDK + c], acc);
    sm.S[r * SM::LDK + c] = acc;
  }
  __syncthreads();
}

__device__ __forceinline__ float cta_sum(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int w = 0; w < NT / 32; ++w) t += red[w];
  return t;
}

// grid (D / RS, nh, B).  states != null: the state slice at the start of every block is written to
// states[b, h, n, row, :].  S_out may be null (the backward's forward sweep).
template <int D>
__global__ void __launch_bounds__(NT, 1)
gdn_chunk_fwd_kernel(const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ beta,
                     const float* __restrict__ la, const float* __restrict__ S0, float* __restrict__ S_out,
                     float* __restrict__ states, int C, int nh) {
  extern __shared__ uint8_t raw[];
  Smem<D>& sm = *reinterpret_cast<Smem<D>*>(raw);
  using SM = Smem<D>;
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int row0 = slice * RS, nb = C / L;
  const long long head = ((long long)b * nh + h) * D * D;
  for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
    const int r = idx / D, c = idx - r * D;
    sm.S[r * SM::LDK + c] = S0[head + (long long)(row0 + r) * D + c];
  }
  __syncthreads();
  for (int n = 0; n < nb; ++n) {
    if (states) {
      float* dst = states + (((long long)b * nh + h) * nb + n) * D * D;
      for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
        const int r = idx / D, c = idx - r * D;
        dst[(long long)(row0 + r) * D + c] = sm.S[r * SM::LDK + c];
      }
    }
    block_forward_parts<D>(sm, k, v, beta, la, (long long)b * C + (long long)n * L, nh, h, row0);
    block_state_update<D>(sm);
  }
  if (S_out) {
    for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
      const int r = idx / D, c = idx - r * D;
      S_out[head + (long long)(row0 + r) * D + c] = sm.S[r * SM::LDK + c];
    }
  }
}

// Backward over the blocks in reverse.  states [B, nh, nb, D, D] from the forward sweep; gS [B, nh, D, D] the gradient
// w.r.t. the chunk's final state.  Outputs: dk_part [D / RS, B, C, nh, D], dv [B, C, nh, D], dbeta_part / dla_part
// [D / RS, B, C, nh], dS0 [B, nh, D, D].
template <int D>
__global__ void __launch_bounds__(NT, 1)
gdn_chunk_bwd_kernel(const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ beta,
                     const float* __restrict__ la, const float* __restrict__ states, const float* __restrict__ gS,
                     float* __restrict__ dk_part, float* __restrict__ dv, float* __restrict__ dbeta_part,
                     float* __restrict__ dla_part, float* __restrict__ dS0, int B, int C, int nh) {
  extern __shared__ uint8_t raw[];
  Smem<D>& sm = *reinterpret_cast<Smem<D>*>(raw);
  using SM = Smem<D>;
  const int slice = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int row0 = slice * RS, nb = C / L;
  const long long head = ((long long)b * nh + h) * D * D;
  for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
    const int r = idx / D, c = idx - r * D;
    sm.G[r * SM::LDK + c] = gS[head + (long long)(row0 + r) * D + c];
  }
  for (int n = nb - 1; n >= 0; --n) {
    const long long tok0 = (long long)b * C + (long long)n * L;
    const float* st = states + (((long long)b * nh + h) * nb + n) * D * D;
    __syncthreads();
    for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
      const int r = idx / D, c = idx - r * D;
      sm.S[r * SM::LDK + c] = st[(long long)(row0 + r) * D + c];
    }
    __syncthreads();
    block_forward_parts<D>(sm, k, v, beta, la, tok0, nh, h, row0);      // K, M, A, T, P, W, U, beta, g, eg, dec
    const float egl = sm.eg[L - 1];
    // dU = diag(dec) K G^T   [L, RS];   X = dK(part) = diag(dec) (U G)   [L, D];   q_i = <K_i, X_i> feeds g
    mm<false>(sm.dU, SM::LDR, sm.K, SM::LDK, 1, sm.G, 1, SM::LDK, L, RS, D);
    mm<false>(sm.X, SM::LDK, sm.U, SM::LDR, 1, sm.G, SM::LDK, 1, L, D, RS);
    if (threadIdx.x < L) { sm.dg[threadIdx.x] = 0.f; sm.dbeta[threadIdx.x] = 0.f; }
    __syncthreads();
    for (int idx = threadIdx.x; idx < L * RS; idx += NT) {
      const int i = idx / RS;
      sm.dU[i * SM::LDR + (idx - i * RS)] *= sm.dec[i];
    }
    for (int idx = threadIdx.x; idx < L * D; idx += NT) {
      const int i = idx / D;
      sm.X[i * SM::LDK + (idx - i * D)] *= sm.dec[i];
    }
    // d gL from the decayed carry: e^{gL} <G, S>
    float part = 0.f;
    for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
      const int r = idx / D, c = idx - r * D;
      part = fmaf(sm.G[r * SM::LDK + c], sm.S[r * SM::LDK + c], part);
    }
    const float dgl_carry = egl * cta_sum(part, sm.red);               // (contains the barrier the scalings above need)
    // q_i = <K_i, X_i>:  d(gL - g_i) = q_i
    if (threadIdx.x < L) {
      const int i = threadIdx.x;
      float q = 0.f;
      for (int c = 0; c < D; ++c) q = fmaf(sm.K[i * SM::LDK + c], sm.X[i * SM::LDK + c], q);
      sm.dg[i] -= q;
      sm.dec[i] = q;                                                    // dec is no longer needed: keep q for the gL sum
    }
    // dR = T^T dU   [L, RS]
    mm<false>(sm.dR, SM::LDR, sm.T, 1, SM::LDL, sm.dU, SM::LDR, 1, L, RS, L);
    __syncthreads();
    if (threadIdx.x == 0) {
      float s = dgl_carry;
      for (int i = 0; i < L; ++i) s += sm.dec[i];
      sm.dg[L - 1] += s;
    }
    // dA = -strict_lower(dR U^T)   [L, L]
    mm<false>(sm.dA, SM::LDL, sm.dR, SM::LDR, 1, sm.U, 1, SM::LDR, L, L, RS, -1.f);
    __syncthreads();
    // d beta_i += <dR_i, W_i>;  dW = beta dR (= dV);  dP = -e^g dW;  d g_i += <dW_i, -e^{g_i} P_i>
    if (threadIdx.x < L) {
      const int i = threadIdx.x;
      float db = 0.f, dgi = 0.f;
      for (int r = 0; r < RS; ++r) {
        const float dr = sm.dR[i * SM::LDR + r];
        db = fmaf(dr, sm.W[i * SM::LDR + r], db);
        dgi = fmaf(sm.beta[i] * dr, -sm.eg[i] * sm.P[i * SM::LDR + r], dgi);
      }
      sm.dbeta[i] += db;
      sm.dg[i] += dgi;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < L * RS; idx += NT) {
      const int i = idx / RS, r = idx - i * RS;
      const float dw = sm.beta[i] * sm.dR[i * SM::LDR + r];
      dv[((tok0 + i) * nh + h) * D + row0 + r] = dw;
      sm.dU[i * SM::LDR + r] = -sm.eg[i] * dw;                          // dP, in dU's place
    }
    __syncthreads();
    // dK += dP S   [L, D];   new G = e^{gL} G + dP^T K   [RS, D]
    mm<true>(sm.X, SM::LDK, sm.dU, SM::LDR, 1, sm.S, SM::LDK, 1, L, D, RS);
    for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
      const int r = idx / D, c = idx - r * D;
      float acc = egl * sm.G[r * SM::LDK + c];
#pragma unroll 8
      for (int i = 0; i < L; ++i) acc = fmaf(sm.dU[i * SM::LDR + r], sm.K[i * SM::LDK + c], acc);
      sm.G[r * SM::LDK + c] = acc;
    }
    // through A = strict_lower(beta_i M_ij Gamma_ij):  E = dA .* A feeds g and beta;  dM = dA .* beta_i Gamma_ij
    __syncthreads();
    if (threadIdx.x < L) {
      const int i = threadIdx.x;
      float row = 0.f, col = 0.f, db = 0.f;
      for (int j = 0; j < i; ++j) {
        const float da = sm.dA[i * SM::LDL + j];
        row = fmaf(da, sm.A[i * SM::LDL + j], row);
        db = fmaf(da, sm.M[i * SM::LDL + j] * __expf(sm.g[i] - sm.g[j]), db);
      }
      for (int j = i + 1; j < L; ++j) col = fmaf(sm.dA[j * SM::LDL + i], sm.A[j * SM::LDL + i], col);
      sm.dg[i] += row - col;
      sm.dbeta[i] += db;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < L * L; idx += NT) {
      const int i = idx / L, j = idx - i * L;
      sm.dA[i * SM::LDL + j] = (i > j) ? sm.dA[i * SM::LDL + j] * sm.beta[i] * __expf(sm.g[i] - sm.g[j]) : 0.f;     // dM (lower)
    }
    __syncthreads();
    // dK += dM K + dM^T K
    mm<true>(sm.X, SM::LDK, sm.dA, SM::LDL, 1, sm.K, SM::LDK, 1, L, D, L);
    __syncthreads();
    mm<true>(sm.X, SM::LDK, sm.dA, 1, SM::LDL, sm.K, SM::LDK, 1, L, D, L);
    __syncthreads();
    // g is a running sum of log a inside the block: d log a_j = sum_{i >= j} d g_i
    if (threadIdx.x == 0) {
      float run = 0.f;
      for (int i = L - 1; i >= 0; --i) { run += sm.dg[i]; sm.dg[i] = run; }
    }
    __syncthreads();
    const long long part_tok = ((long long)slice * B * C + tok0);
    for (int idx = threadIdx.x; idx < L * D; idx += NT) {
      const int i = idx / D, c = idx - i * D;
      dk_part[((part_tok + i) * nh + h) * D + c] = sm.X[i * SM::LDK + c];
    }
    if (threadIdx.x < L) {
      dbeta_part[(part_tok + threadIdx.x) * nh + h] = sm.dbeta[threadIdx.x];
      dla_part[(part_tok + threadIdx.x) * nh + h] = sm.dg[threadIdx.x];
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < RS * D; idx += NT) {
    const int r = idx / D, c = idx - r * D;
    dS0[head + (long long)(row0 + r) * D + c] = sm.G[r * SM::LDK + c];
  }
}

template <int D>
int set_smem(const void* fn) {
  return (int)cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem<D>));
}

}  // namespace

// Bytes of the block-state scratch the backward needs: B * nh * (C / 64) * D * D floats.
extern "C" long long dttt_gdn_chunk_state_elems(int B, int C, int nh, int D) { return (long long)B * nh * (C / L) * D * D; }

// k, v [B, C, nh, D] f32; beta, log_alpha [B, C, nh] f32; S0, S_out [B, nh, D, D] f32; states (may be null) as above.
// C a multiple of 64, D in {64, 128}.
extern "C" int dttt_gdn_chunk_fwd(const float* k, const float* v, const float* beta, const float* log_alpha, const float* S0,
                                  float* S_out, float* states, int B, int C, int nh, int D, cudaStream_t s) {
  if (C % L || (D != 64 && D != 128) || B <= 0 || nh <= 0) return -2;
  dim3 grid(D / RS, nh, B);
  if (D == 128) {
    static int once = set_smem<128>((const void*)gdn_chunk_fwd_kernel<128>);
    (void)once;
    gdn_chunk_fwd_kernel<128><<<grid, NT, sizeof(Smem<128>), s>>>(k, v, beta, log_alpha, S0, S_out, states, C, nh);
  } else {
    static int once = set_smem<64>((const void*)gdn_chunk_fwd_kernel<64>);
    (void)once;
    gdn_chunk_fwd_kernel<64><<<grid, NT, sizeof(Smem<64>), s>>>(k, v, beta, log_alpha, S0, S_out, states, C, nh);
  }
  return (int)cudaGetLastError();
}

// The gradient of dttt_gdn_chunk_fwd.  `states` must come from a forward call with the same inputs.
extern "C" int dttt_gdn_chunk_bwd(const float* k, const float* v, const float* beta, const float* log_alpha, const float* states,
                                  const float* gS, float* dk_part, float* dv, float* dbeta_part, float* dla_part, float* dS0, int B,
                                  int C, int nh, int D, cudaStream_t s) {
  if (C % L || (D != 64 && D != 128) || B <= 0 || nh <= 0) return -2;
  dim3 grid(D / RS, nh, B);
  if (D == 128) {
    static int once = set_smem<128>((const void*)gdn_chunk_bwd_kernel<128>);
    (void)once;
    gdn_chunk_bwd_kernel<128><<<grid, NT, sizeof(Smem<128>), s>>>(k, v, beta, log_alpha, states, gS, dk_part, dv, dbeta_part, dla_part, dS0, B, C, nh);
  } else {
    static int once = set_smem<64>((const void*)gdn_chunk_bwd_kernel<64>);
    (void)once;
    gdn_chunk_bwd_kernel<64><<<grid, NT, sizeof(Smem<64>), s>>>(k, v, beta, log_alpha, states, gS, dk_part, dv, dbeta_part, dla_part, dS0, B, C, nh);
  }
  return (int)cudaGetLastError();
}
