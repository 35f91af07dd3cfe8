// Second-order elementwise kernels: the derivatives of the RMSNorm backward and of the SwiGLU backward, which the outer
// gradient needs wherever the inner loss's backward passed through a norm or a gated activation (the reference gets
// them from JAX differentiating model.py:123-134 and its SwiGLU twice).
//
// RMSNorm.  With r = rsqrt(mean(x^2) + eps), xh = x r, u = w g the first backward is
//     dx = r (u - xh mean(u xh)),   dw = sum_rows g xh.
// For cotangents c of dx and e of dw (e may be absent), per row alpha = mean(c xh), beta = mean(u xh), gamma = mean(c u),
// v = e g, delta = mean(v xh):
//     grad g = w r (c - xh alpha) + e xh
//     grad x = r^2 ((3 alpha beta - gamma) xh - beta c - alpha u) + r (v - xh delta)
//     grad w = sum_rows g r (c - xh alpha)
// SwiGLU.  With s = sigmoid(g), silu = g s, s1 = s (1 + g (1 - s)), s2 = s (1 - s) (2 + g (1 - 2 s)) the first backward
// is dg = dy u s1, du = dy silu.  For cotangents cg, cu:
//     grad dy = cg u s1 + cu silu,   grad u = cg dy s1,   grad g = cg dy u s2 + cu dy s1.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 t = __bfloat1622float2(p[i]);
    f[2 * i] = t.x; f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) p[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row, the row's three inputs held in registers between the reduction and the outputs (NC 16-byte pieces per lane,
// up to NC = 4).
template <int NC>
__global__ void rmsnorm_bwd2_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const __nv_bfloat16* __restrict__ g,
                                    const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ c, const float* __restrict__ e,
                                    __nv_bfloat16* __restrict__ gg, __nv_bfloat16* __restrict__ gx, float* __restrict__ gw, long long rows, int D) {
  extern __shared__ float sgw[];
  const int lane = threadIdx.x & 31;
  const int nvec = D / 8;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  if (gw) {
    for (int i = threadIdx.x; i < D; i += blockDim.x) sgw[i] = 0.f;
    __syncthreads();
  }
  float acc[NC][8];
#pragma unroll
  for (int j = 0; j < NC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
  const float invD = 1.f / D;
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(g + row * D);
    const uint4* cr = reinterpret_cast<const uint4*>(c + row * D);
    constexpr bool CACHE = NC <= 4;                      // wider rows are read again (from L1 / L2) for the outputs
    uint4 vx[CACHE ? NC : 1], vg[CACHE ? NC : 1], vc[CACHE ? NC : 1];
    if constexpr (CACHE) {
#pragma unroll
      for (int j = 0; j < NC; ++j) {
        const int k = lane + 32 * j;
        const bool in = k < nvec;
        vx[j] = in ? xr[k] : make_uint4(0, 0, 0, 0);
        vg[j] = in ? gr[k] : make_uint4(0, 0, 0, 0);
        vc[j] = in ? cr[k] : make_uint4(0, 0, 0, 0);
      }
    }
    const float r = rstd[row];
    float al = 0.f, be = 0.f, ga = 0.f, de = 0.f;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int k = lane + 32 * j;
      if (k < nvec) {
        float fx[8], fg[8], fc[8];
        unpack8(CACHE ? vx[j] : xr[k], fx); unpack8(CACHE ? vg[j] : gr[k], fg); unpack8(CACHE ? vc[j] : cr[k], fc);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * k], w1 = reinterpret_cast<const float4*>(w)[2 * k + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float ee[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (e) {
          const float4 e0 = reinterpret_cast<const float4*>(e)[2 * k], e1 = reinterpret_cast<const float4*>(e)[2 * k + 1];
          ee[0] = e0.x; ee[1] = e0.y; ee[2] = e0.z; ee[3] = e0.w; ee[4] = e1.x; ee[5] = e1.y; ee[6] = e1.z; ee[7] = e1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = fx[i] * r, u = ww[i] * fg[i];
          al += fc[i] * xh; be += u * xh; ga += fc[i] * u; de += ee[i] * fg[i] * xh;
        }
      }
    }
    al = warp_sum(al) * invD; be = warp_sum(be) * invD; ga = warp_sum(ga) * invD; de = warp_sum(de) * invD;
    uint4* ogg = reinterpret_cast<uint4*>(gg + row * D);
    uint4* ogx = reinterpret_cast<uint4*>(gx + row * D);
    const float k3 = 3.f * al * be - ga;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int k = lane + 32 * j;
      if (k < nvec) {
        float fx[8], fg[8], fc[8], o1[8], o2[8];
        unpack8(CACHE ? vx[j] : xr[k], fx); unpack8(CACHE ? vg[j] : gr[k], fg); unpack8(CACHE ? vc[j] : cr[k], fc);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * k], w1 = reinterpret_cast<const float4*>(w)[2 * k + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
        float ee[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (e) {
          const float4 e0 = reinterpret_cast<const float4*>(e)[2 * k], e1 = reinterpret_cast<const float4*>(e)[2 * k + 1];
          ee[0] = e0.x; ee[1] = e0.y; ee[2] = e0.z; ee[3] = e0.w; ee[4] = e1.x; ee[5] = e1.y; ee[6] = e1.z; ee[7] = e1.w;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = fx[i] * r, u = ww[i] * fg[i];
          const float t = r * (fc[i] - xh * al);
          o1[i] = ww[i] * t + ee[i] * xh;
          o2[i] = r * r * (k3 * xh - be * fc[i] - al * u) + r * (ee[i] * fg[i] - xh * de);
          acc[j][i] += fg[i] * t;
        }
        ogg[k] = pack8(o1);
        ogx[k] = pack8(o2);
      }
    }
  }
  if (gw) {
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int k = lane + 32 * j;
      if (k < nvec) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&sgw[k * 8 + i], acc[j][i]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&gw[i], sgw[i]);
  }
}

__global__ void swiglu_bwd2_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, const uint4* __restrict__ dy,
                                   const uint4* __restrict__ cg, const uint4* __restrict__ cu, uint4* __restrict__ og, uint4* __restrict__ ou,
                                   uint4* __restrict__ ody, long long nvec) {
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < nvec; t += (long long)gridDim.x * blockDim.x) {
    float fg[8], fu[8], fd[8], fcg[8], fcu[8], rg[8], ru[8], rd[8];
    unpack8(g[t], fg); unpack8(u[t], fu); unpack8(dy[t], fd); unpack8(cg[t], fcg); unpack8(cu[t], fcu);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float s = 1.f / (1.f + __expf(-fg[i]));
      const float silu = fg[i] * s;
      const float s1 = s * (1.f + fg[i] * (1.f - s));
      const float s2 = s * (1.f - s) * (2.f + fg[i] * (1.f - 2.f * s));
      rd[i] = fcg[i] * fu[i] * s1 + fcu[i] * silu;
      ru[i] = fcg[i] * fd[i] * s1;
      rg[i] = fd[i] * (fcg[i] * fu[i] * s2 + fcu[i] * s1);
    }
    og[t] = pack8(rg); ou[t] = pack8(ru); ody[t] = pack8(rd);
  }
}

}  // namespace

// x, g, c: bf16 [rows, D]; w: f32 [D]; rstd: f32 [rows]; e: f32 [D] or null; outputs grad_g, grad_x bf16 [rows, D];
// grad_w: f32 [D] ACCUMULATED (zero it first) or null.  D a multiple of 8, at most 8192.
extern "C" int dttt_rmsnorm_bwd2(const void* x, const float* w, const void* g, const float* rstd, const void* c, const float* e, void* gg,
                                 void* gx, float* gw, long long rows, int D, cudaStream_t s) {
  if (D % 8 || D > 8192 || rows <= 0) return -2;
  const int wpb = 8;
  long long blocks = (rows + wpb - 1) / wpb;
  int grid = (int)(blocks > 148 * 4 ? 148 * 4 : blocks);
  const int chunks = (D / 8 + 31) / 32;
  size_t smem = (size_t)D * sizeof(float);
#define LAUNCH(NC) rmsnorm_bwd2_kernel<NC><<<grid, wpb * 32, smem, s>>>((const __nv_bfloat16*)x, w, (const __nv_bfloat16*)g, rstd, \
    (const __nv_bfloat16*)c, e, (__nv_bfloat16*)gg, (__nv_bfloat16*)gx, gw, rows, D)
  if (chunks <= 1) LAUNCH(1);
  else if (chunks <= 2) LAUNCH(2);
  else if (chunks <= 4) LAUNCH(4);
  else if (chunks <= 8) LAUNCH(8);
  else if (chunks <= 16) LAUNCH(16);
  else LAUNCH(32);
#undef LAUNCH
  return (int)cudaGetLastError();
}

// g, u, dy, cg, cu: bf16 [n] (n a multiple of 8); outputs grad_g, grad_u, grad_dy like them.
extern "C" int dttt_swiglu_bwd2(const void* g, const void* u, const void* dy, const void* cg, const void* cu, void* og, void* ou, void* ody,
                                long long n, cudaStream_t s) {
  if (n % 8 || n <= 0) return -2;
  const long long nvec = n / 8;
  long long blocks = (nvec + 255) / 256;
  int grid = (int)(blocks > 148 * 16 ? 148 * 16 : blocks);
  swiglu_bwd2_kernel<<<grid, 256, 0, s>>>((const uint4*)g, (const uint4*)u, (const uint4*)dy, (const uint4*)cg, (const uint4*)cu, (uint4*)og,
                                         (uint4*)ou, (uint4*)ody, nvec);
  return (int)cudaGetLastError();
}
