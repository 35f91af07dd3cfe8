// Row stage of the second-order attention backward (the derivative of the first backward, taken by the outer
// gradient of the test-time-training objective through every inner write; the reference gets it from JAX's
// autodiff of its attention, attention.py:181-201).
//
// The first backward is  dS = P o (dP - D),  dQ = scale dS K,  dK = scale dS^T Q,  dV = P^T dO  with
// P = softmax(scale Q K^T), dP = dO V^T, D = rowsum(P o dP).  For cotangents (gQ, gK, gV) of (dQ, dK, dV):
//   gdS = scale (gQ K^T + Q gK^T)          X = dO gV^T
//   E   = rowsum(P o gdS)                  F = rowsum(P o X) + rowsum(gdS o dS) - E D
//   gdP = P o (gdS - E)                    gS = P o X + gdS o dS - E (P o dP) - F P
// and the results are products of P, dS, gdP, gS with the small operands.  The four score-shaped products
// (Q K^T, dO V^T, gQ K^T + Q gK^T, dO gV^T) come from the tensor-core GEMM in f32; this kernel reads one row
// of each from DRAM once, forms the three row sums in one sweep, and writes the four bf16 operand matrices
// of the output GEMMs (dS and gS pre-multiplied by `scale`).  One CTA of 256 threads per row, NV float4 per
// thread and array.  P and gdS stay in registers across the row reduction; dP and X are read again after it
// (a few microseconds later, from L2) so that the register file holds two rows per SM and the load, compute
// and store phases of neighbouring rows overlap.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ uint2 pack4(float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&lo);
  r.y = *reinterpret_cast<uint32_t*>(&hi);
  return r;
}

template <int NV>
__global__ void __launch_bounds__(256, 2) attn_bwd2_rows_kernel(
    const float* __restrict__ S, const float* __restrict__ dP, const float* __restrict__ gdS, const float* __restrict__ X,
    const float* __restrict__ lse, const float* __restrict__ delta, __nv_bfloat16* __restrict__ P, __nv_bfloat16* __restrict__ dSo,
    __nv_bfloat16* __restrict__ gdPo, __nv_bfloat16* __restrict__ gSo, int Kn, int C, int causal, float scale) {
  const long long row = blockIdx.x;
  const long long base = row * (long long)Kn;
  const int c = (int)(row % C);
  const int last = causal ? c + (Kn - C) : Kn - 1;             // newest key this query row sees
  const float L = lse[row], D = delta[row];
  float p[NV][4], gs[NV][4];
  float e = 0.f, a = 0.f, b = 0.f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int col = (threadIdx.x + v * 256) * 4;
    if (col < Kn) {
      const float4 s4 = __ldcs(reinterpret_cast<const float4*>(S + base + col));
      const float4 d4 = __ldg(reinterpret_cast<const float4*>(dP + base + col));
      const float4 g4 = __ldcs(reinterpret_cast<const float4*>(gdS + base + col));
      const float4 x4 = __ldg(reinterpret_cast<const float4*>(X + base + col));
      const float sv[4] = {s4.x, s4.y, s4.z, s4.w}, dv[4] = {d4.x, d4.y, d4.z, d4.w};
      const float gv[4] = {g4.x, g4.y, g4.z, g4.w}, xv[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pi = (col + i <= last) ? __expf(sv[i] * scale - L) : 0.f;
        const float gi = gv[i] * scale;
        p[v][i] = pi; gs[v][i] = gi;
        e += pi * gi;
        a += pi * xv[i];
        b += gi * pi * (dv[i] - D);
      }
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) { p[v][i] = 0.f; gs[v][i] = 0.f; }
    }
  }
  __shared__ float red[3][8];
  e = warp_sum(e); a = warp_sum(a); b = warp_sum(b);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) { red[0][warp] = e; red[1][warp] = a; red[2][warp] = b; }
  __syncthreads();
  float E = 0.f, A = 0.f, Bs = 0.f;
#pragma unroll
  for (int w = 0; w < 8; ++w) { E += red[0][w]; A += red[1][w]; Bs += red[2][w]; }
  const float F = A + Bs - E * D;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int col = (threadIdx.x + v * 256) * 4;
    if (col < Kn) {
      const float4 d4 = __ldcs(reinterpret_cast<const float4*>(dP + base + col));
      const float4 x4 = __ldcs(reinterpret_cast<const float4*>(X + base + col));
      const float dv[4] = {d4.x, d4.y, d4.z, d4.w}, xv[4] = {x4.x, x4.y, x4.z, x4.w};
      float o0[4], o1[4], o2[4], o3[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float pi = p[v][i], ds = pi * (dv[i] - D);
        o0[i] = pi;
        o1[i] = ds * scale;
        o2[i] = pi * (gs[v][i] - E);
        o3[i] = (pi * xv[i] + gs[v][i] * ds - E * pi * dv[i] - F * pi) * scale;
      }
      *reinterpret_cast<uint2*>(P + base + col) = pack4(o0[0], o0[1], o0[2], o0[3]);
      *reinterpret_cast<uint2*>(dSo + base + col) = pack4(o1[0], o1[1], o1[2], o1[3]);
      *reinterpret_cast<uint2*>(gdPo + base + col) = pack4(o2[0], o2[1], o2[2], o2[3]);
      *reinterpret_cast<uint2*>(gSo + base + col) = pack4(o3[0], o3[1], o3[2], o3[3]);
    }
  }
}

template <int NV>
int launch_rows(const float* S, const float* dP, const float* gdS, const float* X, const float* lse, const float* delta, void* P, void* dS,
                void* gdP, void* gS, long long rows, int Kn, int C, int causal, float scale, cudaStream_t s) {
  attn_bwd2_rows_kernel<NV><<<(unsigned)rows, 256, 0, s>>>(S, dP, gdS, X, lse, delta, (__nv_bfloat16*)P, (__nv_bfloat16*)dS, (__nv_bfloat16*)gdP,
                                                            (__nv_bfloat16*)gS, Kn, C, causal, scale);
  return (int)cudaGetLastError();
}

}  // namespace

// S, dP, gdS, X: f32 [rows, Kn] contiguous (unscaled scores, dO V^T, unscaled gQ K^T + Q gK^T, dO gV^T); lse, delta: f32 [rows];
// P, dS, gdP, gS: bf16 [rows, Kn] outputs.  Row r belongs to query position r % C of its chunk; `causal` aligns the triangle to
// the end of the key axis.  Kn a multiple of 4, at most 10240; rows below 2^31.  Returns 0, -1 for an unsupported shape, or a
// CUDA error code.
extern "C" int dttt_attn_bwd2_rows(const float* S, const float* dP, const float* gdS, const float* X, const float* lse, const float* delta,
                                   void* P, void* dS, void* gdP, void* gS, long long rows, int Kn, int C, int causal, float scale,
                                   void* stream) {
  if (rows <= 0 || rows >= (1ll << 31) || Kn <= 0 || Kn % 4 || Kn > 10240 || C <= 0) return -1;
  cudaStream_t s = (cudaStream_t)stream;
  const int nv = (Kn + 1023) / 1024;
#define DTTT_ROWS_CASE(N) case N: return launch_rows<N>(S, dP, gdS, X, lse, delta, P, dS, gdP, gS, rows, Kn, C, causal, scale, s);
  switch (nv) {
    DTTT_ROWS_CASE(1) DTTT_ROWS_CASE(2) DTTT_ROWS_CASE(3) DTTT_ROWS_CASE(4) DTTT_ROWS_CASE(5)
    DTTT_ROWS_CASE(6) DTTT_ROWS_CASE(7) DTTT_ROWS_CASE(8) DTTT_ROWS_CASE(9) DTTT_ROWS_CASE(10)
  }
#undef DTTT_ROWS_CASE
  return -1;
}
