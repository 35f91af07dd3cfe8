// Objective-side and embedding kernels.
//
//   embed_gather       out[i, :] = table[ids[i], :]                      (bf16 rows, 16-byte accesses)
//   embed_scatter_f32  dE[ids[i], :] += dh[i, :] in f32                   (reference src/ttt/model.py:534-542: the
//                      tied embedding's gradient must be summed in f32 -- the mask row is hit thousands of times)
//   cart_band          out[b, t] = sum_d kernel[d + W] x[b, t + d]        (the CART visible-neighbour density,
//                      reference src/ttt/objective.py:91-109; a 2 W + 1 tap correlation, zero padded)
//   threefry_uniform   u[r, i] = uniform(key_r, i) in [0, 1) from threefry2x32 counters (the partitionable
//                      derivation of utils/rng.py: bits = y0 ^ y1 of threefry(key, (i >> 32, i & 0xffffffff))),
//                      optionally compared against a per-row threshold to give the mask directly
//                      (reference src/ttt/objective.py:54-77)
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

namespace {

__global__ void embed_gather_kernel(const __nv_bfloat16* __restrict__ table, const long long* __restrict__ ids,
                                    __nv_bfloat16* __restrict__ out, long long n, int H) {
  const int vec = H / 8;                                   // 16-byte vectors per row
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n * vec; g += (long long)gridDim.x * blockDim.x) {
    const long long row = g / vec;
    const int c = (int)(g - row * vec);
    reinterpret_cast<uint4*>(out + row * H)[c] = reinterpret_cast<const uint4*>(table + ids[row] * H)[c];
  }
}

__global__ void embed_scatter_kernel(const __nv_bfloat16* __restrict__ dh, const long long* __restrict__ ids,
                                     float* __restrict__ dE, long long n, int H) {
  const int vec = H / 4;                                   // four floats per reduction
  for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n * vec; g += (long long)gridDim.x * blockDim.x) {
    const long long row = g / vec;
    const int c = (int)(g - row * vec);
    const uint2 v = reinterpret_cast<const uint2*>(dh + row * H)[c];
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    float* dst = dE + ids[row] * H + 4 * c;
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y) : "memory");
  }
}

// One block per (row b, tile of 256 outputs): the tile's inputs x[t0 - W, t0 + 256 + W) and the kernel sit in shared memory.
__global__ void cart_band_kernel(const float* __restrict__ x, const float* __restrict__ kernel, float* __restrict__ out, int T, int W) {
  extern __shared__ float sm[];
  float* sk = sm;                                          // [2 W + 1]
  float* sx = sm + 2 * W + 1;                              // [256 + 2 W]
  const int b = blockIdx.y, t0 = blockIdx.x * 256;
  const float* xb = x + (long long)b * T;
  for (int i = threadIdx.x; i < 2 * W + 1; i += blockDim.x) sk[i] = kernel[i];
  for (int i = threadIdx.x; i < 256 + 2 * W; i += blockDim.x) {
    const int t = t0 - W + i;
    sx[i] = (t >= 0 && t < T) ? xb[t] : 0.f;
  }
  __syncthreads();
  const int t = t0 + threadIdx.x;
  if (t < T) {
    float a0 = 0.f, a1 = 0.f;
    int d = 0;
    for (; d + 1 < 2 * W + 1; d += 2) {
      a0 = fmaf(sk[d], sx[threadIdx.x + d], a0);
      a1 = fmaf(sk[d + 1], sx[threadIdx.x + d + 1], a1);
    }
    if (d < 2 * W + 1) a0 = fmaf(sk[d], sx[threadIdx.x + d], a0);
    out[(long long)b * T + t] = a0 + a1;
  }
}

__device__ __forceinline__ uint32_t rotl32(uint32_t x, int r) { return (x << r) | (x >> (32 - r)); }

__device__ __forceinline__ uint32_t threefry_bits(uint32_t k0, uint32_t k1, uint32_t c0, uint32_t c1) {
  const uint32_t ks[3] = {k0, k1, k0 ^ k1 ^ 0x1BD11BDAu};
  const int rot[2][4] = {{13, 15, 26, 6}, {17, 29, 16, 24}};
  uint32_t x0 = c0 + ks[0], x1 = c1 + ks[1];
#pragma unroll
  for (int i = 0; i < 5; ++i) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      x0 += x1;
      x1 = rotl32(x1, rot[i % 2][j]) ^ x0;
    }
    x0 += ks[(i + 1) % 3];
    x1 += ks[(i + 2) % 3] + (uint32_t)(i + 1);
  }
  return x0 ^ x1;
}

// keys [R, 2] (int64 holding 32-bit halves); u [R, n] f32 and / or mask [R, n] u8 = u < thresh[r]
__global__ void threefry_uniform_kernel(const long long* __restrict__ keys, long long n, float* __restrict__ u,
                                        const float* __restrict__ thresh, uint8_t* __restrict__ mask) {
  const int r = blockIdx.y;
  const uint32_t k0 = (uint32_t)keys[2 * r], k1 = (uint32_t)keys[2 * r + 1];
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const uint32_t bits = threefry_bits(k0, k1, (uint32_t)(i >> 32), (uint32_t)i);
    const float f = __uint_as_float((bits >> 9) | 0x3F800000u) - 1.0f;
    if (u) u[(long long)r * n + i] = f;
    if (mask) mask[(long long)r * n + i] = f < thresh[r] ? 1 : 0;
  }
}

inline int blocks_for(long long work, int block, int cap) {
  long long g = (work + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" int dttt_embed_gather(const void* table, const long long* ids, void* out, long long n, int H, cudaStream_t s) {
  if (H % 8) return -2;
  embed_gather_kernel<<<blocks_for(n * (H / 8), 256, 148 * 16), 256, 0, s>>>((const __nv_bfloat16*)table, ids, (__nv_bfloat16*)out, n, H);
  return (int)cudaGetLastError();
}

extern "C" int dttt_embed_scatter_f32(const void* dh, const long long* ids, float* dE, long long n, int H, cudaStream_t s) {
  if (H % 4) return -2;
  embed_scatter_kernel<<<blocks_for(n * (H / 4), 256, 148 * 16), 256, 0, s>>>((const __nv_bfloat16*)dh, ids, dE, n, H);
  return (int)cudaGetLastError();
}

extern "C" int dttt_cart_band(const float* x, const float* kernel, float* out, int B, int T, int W, cudaStream_t s) {
  const size_t smem = (size_t)(2 * W + 1 + 256 + 2 * W) * sizeof(float);
  if (smem > 48 * 1024) return -2;
  dim3 grid((T + 255) / 256, B);
  cart_band_kernel<<<grid, 256, smem, s>>>(x, kernel, out, T, W);
  return (int)cudaGetLastError();
}

extern "C" int dttt_threefry_uniform(const long long* keys, int rows, long long n, float* u, const float* thresh, void* mask,
                                     cudaStream_t s) {
  dim3 grid(blocks_for(n, 256, 148 * 4), rows);
  threefry_uniform_kernel<<<grid, 256, 0, s>>>(keys, n, u, thresh, (uint8_t*)mask);
  return (int)cudaGetLastError();
}
