// Row kernels of the second-order linear + cross-entropy (the derivative of the cross-entropy backward, which the
// outer gradient needs through the inner loss of every write; the reference differentiates its fused
// cross-entropy's custom VJP a second time, fused_ce.py:84-121).
//
// The first backward is  g_h = gw (p E - E_y),  p = softmax(h E^T),  gw = g w.  For a cotangent c of g_h, with
// u = c E^T and ubar = rowsum(p o u):
//   r = gw p o (u - ubar)      grad h = r E      grad E = r^T h + d^T c,   d = gw (p - onehot(y))
// `rowdot` forms ubar from the f32 logits z and u; `make` writes r and d (bf16) for the three output products.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(256) ce_bwd2_rowdot_kernel(const float* __restrict__ z, const float* __restrict__ u,
                                                             const float* __restrict__ lse, float* __restrict__ ubar, int W, long long ld) {
  const long long row = blockIdx.x;
  const float* zr = z + row * ld;
  const float* ur = u + row * ld;
  const float L = lse[row];
  float acc = 0.f;
  for (int col = threadIdx.x * 4; col < W; col += 1024) {
    const float4 a = *reinterpret_cast<const float4*>(zr + col);
    const float4 b = *reinterpret_cast<const float4*>(ur + col);
    acc += __expf(a.x - L) * b.x + __expf(a.y - L) * b.y + __expf(a.z - L) * b.z + __expf(a.w - L) * b.w;
  }
  __shared__ float red[8];
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    ubar[row] = t;
  }
}

__device__ __forceinline__ uint2 pack4(float a, float b, float c, float d) {
  __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 r;
  r.x = *reinterpret_cast<uint32_t*>(&lo);
  r.y = *reinterpret_cast<uint32_t*>(&hi);
  return r;
}

__global__ void __launch_bounds__(256) ce_bwd2_make_kernel(const float* __restrict__ z, const float* __restrict__ u, const float* __restrict__ lse,
                                                           const float* __restrict__ ubar, const float* __restrict__ gw,
                                                           const int* __restrict__ targets, __nv_bfloat16* __restrict__ r,
                                                           __nv_bfloat16* __restrict__ d, int W, long long ld) {
  const long long row = blockIdx.x;
  const float* zr = z + row * ld;
  const float* ur = u + row * ld;
  const float L = lse[row], ub = ubar[row], c = gw[row];
  const int y = targets[row];
  for (int col = threadIdx.x * 4; col < W; col += 1024) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(zr + col));
    const float4 b = __ldcs(reinterpret_cast<const float4*>(ur + col));
    const float p0 = __expf(a.x - L), p1 = __expf(a.y - L), p2 = __expf(a.z - L), p3 = __expf(a.w - L);
    *reinterpret_cast<uint2*>(r + row * ld + col) = pack4(c * p0 * (b.x - ub), c * p1 * (b.y - ub), c * p2 * (b.z - ub), c * p3 * (b.w - ub));
    *reinterpret_cast<uint2*>(d + row * ld + col) = pack4(c * (p0 - (col == y ? 1.f : 0.f)), c * (p1 - (col + 1 == y ? 1.f : 0.f)),
                                                          c * (p2 - (col + 2 == y ? 1.f : 0.f)), c * (p3 - (col + 3 == y ? 1.f : 0.f)));
  }
}

}  // namespace

// z, u: f32 [N, W] with row stride ld (elements); lse: f32 [N]; ubar: f32 [N] output.  W and ld multiples of 4, 16-byte aligned bases.
extern "C" int dttt_ce_bwd2_rowdot(const float* z, const float* u, const float* lse, float* ubar, long long N, int W, long long ld, void* stream) {
  if (N <= 0 || N >= (1ll << 31) || W <= 0 || W % 4 || ld % 4) return -1;
  ce_bwd2_rowdot_kernel<<<(unsigned)N, 256, 0, (cudaStream_t)stream>>>(z, u, lse, ubar, W, ld);
  return (int)cudaGetLastError();
}

// r, d: bf16 [N, W] outputs with the same row stride ld; gw: f32 [N]; targets: int32 [N] (column of the label).
extern "C" int dttt_ce_bwd2_make(const float* z, const float* u, const float* lse, const float* ubar, const float* gw, const int* targets,
                                 void* r, void* d, long long N, int W, long long ld, void* stream) {
  if (N <= 0 || N >= (1ll << 31) || W <= 0 || W % 4 || ld % 4) return -1;
  ce_bwd2_make_kernel<<<(unsigned)N, 256, 0, (cudaStream_t)stream>>>(z, u, lse, ubar, gw, targets, (__nv_bfloat16*)r, (__nv_bfloat16*)d, W, ld);
  return (int)cudaGetLastError();
}
