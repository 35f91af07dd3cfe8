// Gated delta rule, token-sequential, one chunk per launch (forward / no-grad use):
//
//   S_t = a_t S_{t-1} + b_t (v_t - a_t S_{t-1} k_t) k_t^T          S [dv, dk] per (sequence, head), f32
//
// (reference src/ttt/gdn.py:106-123; its plain loop :125-136 is the oracle).  One CTA owns the state of one (sequence,
// head): 256 threads, dv rows x (256 / dv) threads per row, each thread keeping its dk / (256 / dv) state elements in
// registers for the whole chunk.  Per token a thread decays its elements, forms its part of the row's dot product with
// k_t, the partial sums are combined by warp shuffles, and the rank-one correction is added: three FMA passes over the
// registers and one shuffle tree, nothing leaves the register file until the chunk is done.  k, v, a, b of 32 tokens at a
// time are staged through shared memory.  Exact f32 arithmetic in the order of the recurrence.
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

constexpr int TOK = 32;      // tokens staged per tile

template <int D>             // D = dv = dk (64 or 128)
__global__ void __launch_bounds__(256, 1)
gdn_update_kernel(const float* __restrict__ k, const float* __restrict__ v, const float* __restrict__ beta,
                  const float* __restrict__ log_alpha, const float* __restrict__ S0, float* __restrict__ S_out, int C, int nh) {
  constexpr int TPR = 256 / D;                 // threads per state row
  constexpr int EPT = D / TPR;                 // state elements per thread
  __shared__ float sk[TOK][D];
  __shared__ float sv[TOK][D];
  __shared__ float sa[TOK], sb[TOK];
  const int h = blockIdx.x, b = blockIdx.y;
  const int row = threadIdx.x / TPR, part = threadIdx.x % TPR;
  const long long st_off = (((long long)b * nh + h) * D + row) * D + part * EPT;
  float S[EPT];
#pragma unroll
  for (int e = 0; e < EPT; ++e) S[e] = S0[st_off + e];
  for (int t0 = 0; t0 < C; t0 += TOK) {
    const int nt = min(TOK, C - t0);
    __syncthreads();
    for (int i = threadIdx.x; i < nt * D; i += 256) {
      const int t = i / D, e = i - t * D;
      const long long src = (((long long)b * C + t0 + t) * nh + h) * D + e;
      sk[t][e] = k[src];
      sv[t][e] = v[src];
    }
    if (threadIdx.x < nt) {
      const long long src = ((long long)b * C + t0 + threadIdx.x) * nh + h;
      sa[threadIdx.x] = __expf(log_alpha[src]);
      sb[threadIdx.x] = beta[src];
    }
    __syncthreads();
    for (int t = 0; t < nt; ++t) {
      const float a = sa[t], bt = sb[t];
      const float* kt = &sk[t][part * EPT];
      float dot = 0.f;
#pragma unroll
      for (int e = 0; e < EPT; ++e) {
        S[e] *= a;
        dot = fmaf(S[e], kt[e], dot);
      }
#pragma unroll
      for (int o = TPR / 2; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float c = bt * (sv[t][row] - dot);
#pragma unroll
      for (int e = 0; e < EPT; ++e) S[e] = fmaf(c, kt[e], S[e]);
    }
  }
#pragma unroll
  for (int e = 0; e < EPT; ++e) S_out[st_off + e] = S[e];
}

}  // namespace

// k, v [B, C, nh, D] f32, beta / log_alpha [B, C, nh] f32, S0 / S_out [B, nh, D, D] f32 (S_out may alias S0); D in {64, 128}.
extern "C" int dttt_gdn_update(const float* k, const float* v, const float* beta, const float* log_alpha, const float* S0,
                               float* S_out, int B, int C, int nh, int D, cudaStream_t s) {
  dim3 grid(nh, B);
  if (D == 128) gdn_update_kernel<128><<<grid, 256, 0, s>>>(k, v, beta, log_alpha, S0, S_out, C, nh);
  else if (D == 64) gdn_update_kernel<64><<<grid, 256, 0, s>>>(k, v, beta, log_alpha, S0, S_out, C, nh);
  else return -2;
  return (int)cudaGetLastError();
}
