// Bandwidth-bound kernels: RMSNorm (forward / backward), rotary embedding (forward / backward),
// SwiGLU (forward / backward), AdamW on flat f32 shards, and the per-sequence pieces of the inner
// step (sum of squares, scaled update).  bf16 activations, f32 math, 16-byte vector accesses.
// Each launcher is extern "C", takes raw device pointers and a stream, allocates nothing.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <cstdlib>

namespace {

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(p[i]);
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

// ------------------------------------------------------------------ RMSNorm
// One warp per row; D a multiple of 8.  y = w * x * rsqrt(mean(x^2) + eps), f32 math (reference
// src/ttt/model.py:123-134).
template <int NC>                 // 16-byte pieces of a row per lane: the row stays in registers between the two passes
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, long long rows, int D,
                                   float eps) {
  const int lane = threadIdx.x & 31;
  const int nvec = D / 8;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    uint4 v[NC];
#pragma unroll
    for (int j = 0; j < NC; ++j) {                       // every load of the row is in flight before the first use
      const int c = lane + 32 * j;
      v[j] = c < nvec ? xr[c] : make_uint4(0, 0, 0, 0);
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      float f[8];
      unpack8(v[j], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd) rstd[row] = r;
    uint4* yr = reinterpret_cast<uint4*>(y + row * D);
#pragma unroll
    for (int j = 0; j < NC; ++j) {
      const int c = lane + 32 * j;
      if (c < nvec) {
        float f[8];
        unpack8(v[j], f);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * c], w1 = reinterpret_cast<const float4*>(w)[2 * c + 1];
        f[0] *= r * w0.x; f[1] *= r * w0.y; f[2] *= r * w0.z; f[3] *= r * w0.w;
        f[4] *= r * w1.x; f[5] *= r * w1.y; f[6] *= r * w1.z; f[7] *= r * w1.w;
        yr[c] = pack8(f);
      }
    }
  }
}

// dx = r * (w*dy - xhat * mean(w*dy*xhat)),  dw += sum_rows dy * xhat,  xhat = x * r.
// Each warp walks rows; its lane-local dw partials (for the columns it owns) are reduced through shared
// memory per block and added to the f32 dw with one atomic per column per block.
template <int MAXC>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                                   __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, long long rows, int D) {
  extern __shared__ float sdw[];
  const int lane = threadIdx.x & 31;
  const long long warps = (long long)gridDim.x * (blockDim.x >> 5);
  for (int i = threadIdx.x; i < D; i += blockDim.x) sdw[i] = 0.f;
  __syncthreads();
  float acc[MAXC][8];
#pragma unroll
  for (int j = 0; j < MAXC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
  const int nchunk = D / 8;
  for (long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); row < rows; row += warps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * D);
    const uint4* gr = reinterpret_cast<const uint4*>(dy + row * D);
    const float r = rstd[row];
    // rows of up to 2048 elements stay in registers between the reduction and the output (every load in flight at once)
    constexpr bool CACHE = MAXC <= 8;
    uint4 vx[CACHE ? MAXC : 1], vg[CACHE ? MAXC : 1];
    if constexpr (CACHE) {
#pragma unroll
      for (int j = 0; j < MAXC; ++j) {
        const int c = lane + 32 * j;
        vx[j] = c < nchunk ? xr[c] : make_uint4(0, 0, 0, 0);
        vg[j] = c < nchunk ? gr[c] : make_uint4(0, 0, 0, 0);
      }
    }
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunk) {
        float fx[8], fg[8];
        unpack8(CACHE ? vx[j] : xr[c], fx); unpack8(CACHE ? vg[j] : gr[c], fg);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * c], w1 = reinterpret_cast<const float4*>(w)[2 * c + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = fx[i] * r;
          dot += ww[i] * fg[i] * xh;
          acc[j][i] += fg[i] * xh;
        }
      }
    }
    dot = warp_sum(dot) / D;
    uint4* dr = reinterpret_cast<uint4*>(dx + row * D);
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunk) {
        float fx[8], fg[8], o[8];
        unpack8(CACHE ? vx[j] : xr[c], fx); unpack8(CACHE ? vg[j] : gr[c], fg);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * c], w1 = reinterpret_cast<const float4*>(w)[2 * c + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = r * (ww[i] * fg[i] - fx[i] * r * dot);
        dr[c] = pack8(o);
      }
    }
  }
  if (dw) {
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&sdw[c * 8 + i], acc[j][i]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dw[i], sdw[i]);
  }
}

// ------------------------------------------------------------------ rotary embedding
// x [rows, heads, d] -> out; angle = pos[row] * inv_freq[i]; out = x*cos + rot(x)*sin with
// rot(x) = [-x2, x1] (half rotation, reference model.py:111-117).  sign = -1 gives the backward.
// One thread per (row, head, 8-element slice of the first half).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                            const long long* __restrict__ pos, const float* __restrict__ inv_freq, long long rows,
                            int heads, int d, float sign) {
  const int slices = d / 16;                       // 8-element slices in one half
  const long long total = rows * heads * slices;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int sl = (int)(t % slices);
    const long long rh = t / slices;
    const long long row = rh / heads;
    const __nv_bfloat16* base = x + rh * d;
    float a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const uint4*>(base + sl * 8), a);
    unpack8(*reinterpret_cast<const uint4*>(base + d / 2 + sl * 8), b);
    const float p = (float)pos[row];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float s, c;
      sincosf(p * inv_freq[sl * 8 + i], &s, &c);
      s *= sign;
      oa[i] = a[i] * c - b[i] * s;
      ob[i] = b[i] * c + a[i] * s;
    }
    __nv_bfloat16* ob_ = out + rh * d;
    *reinterpret_cast<uint4*>(ob_ + sl * 8) = pack8(oa);
    *reinterpret_cast<uint4*>(ob_ + d / 2 + sl * 8) = pack8(ob);
  }
}

// ------------------------------------------------------------------ SwiGLU
__global__ void swiglu_fwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, uint4* __restrict__ y,
                                  long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float fg[8], fu[8], o[8];
    unpack8(g[i], fg); unpack8(u[i], fu);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = fg[k] / (1.f + __expf(-fg[k])) * fu[k];
    y[i] = pack8(o);
  }
}
__global__ void swiglu_bwd_kernel(const uint4* __restrict__ g, const uint4* __restrict__ u, const uint4* __restrict__ dy,
                                  uint4* __restrict__ dg, uint4* __restrict__ du, long long n8) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (long long)gridDim.x * blockDim.x) {
    float fg[8], fu[8], fd[8], og[8], ou[8];
    unpack8(g[i], fg); unpack8(u[i], fu); unpack8(dy[i], fd);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float s = 1.f / (1.f + __expf(-fg[k]));
      const float silu = fg[k] * s;
      ou[k] = fd[k] * silu;
      og[k] = fd[k] * fu[k] * (s + silu * (1.f - s));
    }
    dg[i] = pack8(og); du[i] = pack8(ou);
  }
}

// ------------------------------------------------------------------ AdamW on a flat f32 range
// g is pre-multiplied by gscale (the clip factor); optax semantics (see optim.py).
__global__ void adamw_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ g, long long n, float lr, float b1, float b2, float eps, float wd,
                             float bc1, float bc2, float gscale) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float gg = g[i] * gscale;
    const float mm = b1 * m[i] + (1.f - b1) * gg;
    const float vv = b2 * v[i] + (1.f - b2) * gg * gg;
    m[i] = mm; v[i] = vv;
    const float pp = p[i];
    const float upd = (mm / bc1) / (sqrtf(vv / bc2) + eps) + wd * pp;
    p[i] = pp - lr * upd;
  }
}

// four elements per thread and iteration (16-byte accesses); n4 = n / 4
__global__ void adamw_kernel_v4(float4* __restrict__ p, float4* __restrict__ m, float4* __restrict__ v,
                                const float4* __restrict__ g, long long n4, float lr, float b1, float b2, float eps, float wd,
                                float bc1, float bc2, float gscale) {
  const float ib1 = 1.f / bc1, ib2 = 1.f / bc2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 g4 = g[i];
    float4 m4 = m[i], v4 = v[i], p4 = p[i];
    const float gg[4] = {g4.x * gscale, g4.y * gscale, g4.z * gscale, g4.w * gscale};
    float* mp = reinterpret_cast<float*>(&m4);
    float* vp = reinterpret_cast<float*>(&v4);
    float* pp = reinterpret_cast<float*>(&p4);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mp[k] = b1 * mp[k] + (1.f - b1) * gg[k];
      vp[k] = b2 * vp[k] + (1.f - b2) * gg[k] * gg[k];
      const float upd = (mp[k] * ib1) / (sqrtf(vp[k] * ib2) + eps) + wd * pp[k];
      pp[k] -= lr * upd;
    }
    m[i] = m4; v[i] = v4; p[i] = p4;
  }
}

// Per-sequence kernels, 16 bytes per access: a row of n elements is n / VEC vectors.
template <typename T> struct Vec;
template <> struct Vec<float> {
  using type = float4;
  __device__ static void load(const float* p, float (&f)[4]) { const float4 v = *reinterpret_cast<const float4*>(p); f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w; }
  __device__ static void store(float* p, const float (&f)[4]) { *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]); }
};
template <> struct Vec<__nv_bfloat16> {
  __device__ static void load(const __nv_bfloat16* p, float (&f)[4]) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  }
  __device__ static void store(__nv_bfloat16* p, const float (&f)[4]) {
    uint2 v;
    *reinterpret_cast<__nv_bfloat162*>(&v.x) = __floats2bfloat162_rn(f[0], f[1]);
    *reinterpret_cast<__nv_bfloat162*>(&v.y) = __floats2bfloat162_rn(f[2], f[3]);
    *reinterpret_cast<uint2*>(p) = v;
  }
};

__device__ __forceinline__ void block_sum_to(float s, float* dst) {
  s = warp_sum(s);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(dst, s);
  }
}

template <typename T>
__global__ void seq_sumsq_v4(const T* __restrict__ x, float* __restrict__ out, long long n) {
  const int b = blockIdx.y;
  const T* xb = x + (long long)b * n;
  float s = 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float f[4];
    Vec<T>::load(xb + i, f);
    s += f[0] * f[0] + f[1] * f[1] + f[2] * f[2] + f[3] * f[3];
  }
  block_sum_to(s, &out[b]);
}

template <typename T>
__global__ void seq_axpy_v4(const float* __restrict__ w, const T* __restrict__ g, const float* __restrict__ coef,
                            float* __restrict__ w_new, __nv_bfloat16* __restrict__ w_lo, long long n) {
  const int b = blockIdx.y;
  const float c = coef[b];
  const long long off = (long long)b * n;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float wv[4], gv[4];
    Vec<float>::load(w + off + i, wv);
    Vec<T>::load(g + off + i, gv);
#pragma unroll
    for (int k = 0; k < 4; ++k) wv[k] -= c * gv[k];
    Vec<float>::store(w_new + off + i, wv);
    if (w_lo) Vec<__nv_bfloat16>::store(w_lo + off + i, wv);
  }
}

template <typename T>
__global__ void seq_dot_v4(const float* __restrict__ a, const T* __restrict__ g, float* __restrict__ out, long long n) {
  const int b = blockIdx.y;
  const long long off = (long long)b * n;
  float s = 0.f;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float av[4], gv[4];
    Vec<float>::load(a + off + i, av);
    Vec<T>::load(g + off + i, gv);
    s += av[0] * gv[0] + av[1] * gv[1] + av[2] * gv[2] + av[3] * gv[3];
  }
  block_sum_to(s, &out[b]);
}

template <typename T>
__global__ void seq_lincomb_v4(const float* __restrict__ a, const T* __restrict__ g, const float* __restrict__ alpha,
                               const float* __restrict__ beta, T* __restrict__ out, long long n) {
  const int b = blockIdx.y;
  const float al = alpha[b], be = beta[b];
  const long long off = (long long)b * n;
  for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (long long)gridDim.x * blockDim.x * 4) {
    float av[4], gv[4];
    Vec<float>::load(a + off + i, av);
    Vec<T>::load(g + off + i, gv);
#pragma unroll
    for (int k = 0; k < 4; ++k) gv[k] = al * av[k] + be * gv[k];
    Vec<T>::store(out + off + i, gv);
  }
}

inline bool vec_ok(long long n, const void* a, const void* b = nullptr, const void* c = nullptr, const void* d = nullptr) {
  auto al = [](const void* p) { return p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  return n % 4 == 0 && al(a) && al(b) && al(c) && al(d);
}

// ------------------------------------------------------------------ inner step pieces (per sequence)
// out[b] += sum over the n elements of sequence b of x^2   (x: [B, n] f32 or bf16)
template <typename T>
__global__ void seq_sumsq_kernel(const T* __restrict__ x, float* __restrict__ out, long long n) {
  const int b = blockIdx.y;
  const T* xb = x + (long long)b * n;
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float f = (float)xb[i];
    s += f * f;
  }
  s = warp_sum(s);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(&out[b], s);
  }
}
// w_new[b, i] = w[b, i] - coef[b] * g[b, i]   (f32 master carry; g f32 or bf16); optional bf16 copy of w_new
template <typename T>
__global__ void seq_axpy_kernel(const float* __restrict__ w, const T* __restrict__ g, const float* __restrict__ coef,
                                float* __restrict__ w_new, __nv_bfloat16* __restrict__ w_lo, long long n) {
  const int b = blockIdx.y;
  const float c = coef[b];
  const long long off = (long long)b * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float r = w[off + i] - c * (float)g[off + i];
    w_new[off + i] = r;
    if (w_lo) w_lo[off + i] = __float2bfloat16(r);
  }
}

// out[b] += sum_i a[b, i] * g[b, i]   (a f32, g f32 or bf16)
template <typename T>
__global__ void seq_dot_kernel(const float* __restrict__ a, const T* __restrict__ g, float* __restrict__ out, long long n) {
  const int b = blockIdx.y;
  const long long off = (long long)b * n;
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    s += a[off + i] * (float)g[off + i];
  s = warp_sum(s);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x < 32) {
    s = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    s = warp_sum(s);
    if (threadIdx.x == 0) atomicAdd(&out[b], s);
  }
}
// out[b, i] = alpha[b] * a[b, i] + beta[b] * g[b, i]   (a f32; g and out f32 or bf16, same type)
template <typename T>
__global__ void seq_lincomb_kernel(const float* __restrict__ a, const T* __restrict__ g, const float* __restrict__ alpha,
                                   const float* __restrict__ beta, T* __restrict__ out, long long n) {
  const int b = blockIdx.y;
  const float al = alpha[b], be = beta[b];
  const long long off = (long long)b * n;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[off + i] = (T)(al * a[off + i] + be * (float)g[off + i]);
}

inline int grid_for(long long n, int block, int cap = 148 * 16) {
  long long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

extern "C" int dttt_rmsnorm_fwd(const void* x, const float* w, void* y, float* rstd, long long rows, int D, float eps,
                                cudaStream_t s) {
  if (D % 8) return -2;
  const int wpb = 8;
  long long blocks = (rows + wpb - 1) / wpb;
  int grid = (int)(blocks > 148 * 32 ? 148 * 32 : (blocks < 1 ? 1 : blocks));
  if (D > 8192) return -2;
  const int nc = (D / 8 + 31) / 32;
#define FWD(NC) rmsnorm_fwd_kernel<NC><<<grid, wpb * 32, 0, s>>>((const __nv_bfloat16*)x, w, (__nv_bfloat16*)y, rstd, rows, D, eps)
  if (nc <= 1) FWD(1);
  else if (nc <= 2) FWD(2);
  else if (nc <= 4) FWD(4);
  else if (nc <= 8) FWD(8);
  else if (nc <= 16) FWD(16);
  else FWD(32);
#undef FWD
  return (int)cudaGetLastError();
}

// The same backward with the rows streamed through shared memory by cp.async: every warp keeps STAGES - 1 rows of x and dy
// in flight while it works on one, and holds nothing of a row in registers between its two passes (the register form
// above needs 228 registers at D = 2048, which leaves eight warps per SM and their loads exposed).  A lane reads back
// exactly the 16-byte pieces it copied itself, so cp.async.wait_group is all the synchronisation the data needs.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <int MAXC, int STAGES>
__global__ void __launch_bounds__(256, 1)
rmsnorm_bwd_async_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const __nv_bfloat16* __restrict__ dy,
                         const float* __restrict__ rstd, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, long long rows, int D) {
  extern __shared__ __align__(16) uint8_t smem_async[];
  float* sdw = reinterpret_cast<float*>(smem_async);
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const int row_bytes = D * 2;
  uint8_t* ring = smem_async + (size_t)D * 4 + (size_t)wid * STAGES * 2 * row_bytes;      // this warp's stages: [x row | dy row]
  const long long warps = (long long)gridDim.x * nw;
  const long long first = (long long)blockIdx.x * nw + wid;
  const int nchunk = D / 8;
  for (int i = threadIdx.x; i < D; i += blockDim.x) sdw[i] = 0.f;
  __syncthreads();
  float acc[MAXC][8];
#pragma unroll
  for (int j = 0; j < MAXC; ++j)
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[j][i] = 0.f;
  auto issue = [&](long long row, int stage) {
    if (row < rows) {
      uint8_t* dst = ring + (size_t)stage * 2 * row_bytes;
      const uint8_t* xs = reinterpret_cast<const uint8_t*>(x + row * D);
      const uint8_t* gs = reinterpret_cast<const uint8_t*>(dy + row * D);
#pragma unroll
      for (int j = 0; j < MAXC; ++j) {
        const int c = lane + 32 * j;
        if (c < nchunk) {
          cp_async16(dst + c * 16, xs + c * 16);
          cp_async16(dst + row_bytes + c * 16, gs + c * 16);
        }
      }
    }
    cp_async_commit();                                       // one group per call, empty past the end: the counting stays uniform
  };
  long long next = first;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) { issue(next, s); next += warps; }
  int stage = 0;
  for (long long row = first; row < rows; row += warps) {
    issue(next, (stage + STAGES - 1) % STAGES);              // the stage read in the previous iteration (its loads have been consumed)
    next += warps;
    cp_async_wait<STAGES - 1>();                             // this row's group has landed
    const uint4* xr = reinterpret_cast<const uint4*>(ring + (size_t)stage * 2 * row_bytes);
    const uint4* gr = reinterpret_cast<const uint4*>(ring + (size_t)stage * 2 * row_bytes + row_bytes);
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunk) {
        float fx[8], fg[8];
        unpack8(xr[c], fx); unpack8(gr[c], fg);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * c], w1 = reinterpret_cast<const float4*>(w)[2 * c + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float xh = fx[i] * r;
          dot += ww[i] * fg[i] * xh;
          acc[j][i] += fg[i] * xh;
        }
      }
    }
    dot = warp_sum(dot) / D;
    uint4* dr = reinterpret_cast<uint4*>(dx + row * D);
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunk) {
        float fx[8], fg[8], o[8];
        unpack8(xr[c], fx); unpack8(gr[c], fg);
        const float4 w0 = reinterpret_cast<const float4*>(w)[2 * c], w1 = reinterpret_cast<const float4*>(w)[2 * c + 1];
        const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = r * (ww[i] * fg[i] - fx[i] * r * dot);
        dr[c] = pack8(o);
      }
    }
    stage = (stage + 1) % STAGES;
  }
  cp_async_wait<0>();
  if (dw) {
#pragma unroll
    for (int j = 0; j < MAXC; ++j) {
      const int c = lane + 32 * j;
      if (c < nchunk) {
#pragma unroll
        for (int i = 0; i < 8; ++i) atomicAdd(&sdw[c * 8 + i], acc[j][i]);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) atomicAdd(&dw[i], sdw[i]);
  }
}

extern "C" int dttt_rmsnorm_bwd(const void* x, const float* w, const void* dy, const float* rstd, void* dx, float* dw,
                                long long rows, int D, cudaStream_t s) {
  if (D % 8 || D > 8192) return -2;
  {
    // Rows of 1024 .. 2048 elements, a chunk's worth of them (measured at D = 2048: 4096 rows 54 -> 38 us, but 49152 rows
    // 161 -> 206 us, crossing near 16 k rows): the streamed form.  DTTT_RMS_BWD_ASYNC=0 turns it off, =2 takes it for any size.
    static const int use_async = getenv("DTTT_RMS_BWD_ASYNC") ? atoi(getenv("DTTT_RMS_BWD_ASYNC")) : 1;
    constexpr int ST = 3, WPB = 8;
    if (use_async && D % 256 == 0 && D >= 1024 && D <= 2048 && rows >= 148 * WPB && (rows <= 12288 || use_async == 2) &&
        ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(dy)) & 15) == 0) {
      const size_t smem = (size_t)D * 4 + (size_t)WPB * ST * 2 * D * 2;
      static bool attr_set[64] = {};
      int dev = 0;
      cudaGetDevice(&dev);
      if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        if (cudaFuncSetAttribute(rmsnorm_bwd_async_kernel<8, ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(8192 + WPB * ST * 2 * 4096)) != cudaSuccess)
          return -3;
        attr_set[dev] = true;
      }
      long long blocks = (rows + WPB - 1) / WPB;
      const int grid = (int)(blocks > 148 ? 148 : blocks);
      rmsnorm_bwd_async_kernel<8, ST><<<grid, WPB * 32, smem, s>>>((const __nv_bfloat16*)x, w, (const __nv_bfloat16*)dy, rstd,
                                                                    (__nv_bfloat16*)dx, dw, rows, D);
      return (int)cudaGetLastError();
    }
  }
  const int wpb = 8;
  long long blocks = (rows + wpb - 1) / wpb;
  const int chunks = (D / 8 + 31) / 32;
  // every block ends with D atomic adds into dw, so no more blocks than can be resident: one per SM from 8 chunks per lane
  // on (228 registers), two at 4, four below
  const int per_sm = chunks >= 8 ? 1 : (chunks >= 4 ? 2 : 4);
  int grid = (int)(blocks > 148 * per_sm ? 148 * per_sm : (blocks < 1 ? 1 : blocks));
  size_t smem = (size_t)D * sizeof(float);
#define LAUNCH(MC) rmsnorm_bwd_kernel<MC><<<grid, wpb * 32, smem, s>>>((const __nv_bfloat16*)x, w, (const __nv_bfloat16*)dy, \
                                                                      rstd, (__nv_bfloat16*)dx, dw, rows, D)
  if (chunks <= 1) LAUNCH(1);
  else if (chunks <= 2) LAUNCH(2);
  else if (chunks <= 4) LAUNCH(4);
  else if (chunks <= 8) LAUNCH(8);
  else if (chunks <= 16) LAUNCH(16);
  else LAUNCH(32);
#undef LAUNCH
  return (int)cudaGetLastError();
}

// The same rotation from a table of (cos, sin) per (row, frequency): the angles depend on the position only, so one table
// serves every head, both of q and k, every layer and the backward of a chunk; the kernel that applies it is a plain
// streaming pass (the direct kernel above spends most of its time in sincosf on angles of up to 1e5 radians).
__global__ void rope_table_kernel(const long long* __restrict__ pos, const float* __restrict__ inv_freq, long long rows,
                                  int half, float2* __restrict__ tab) {
  const long long total = rows * half;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const long long row = t / half;
    const int i = (int)(t - row * half);
    float s, c;
    sincosf((float)pos[row] * inv_freq[i], &s, &c);
    tab[t] = make_float2(c, s);
  }
}

__global__ void rope_apply_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                                  const float2* __restrict__ tab, long long rows, int heads, int d, float sign) {
  const int slices = d / 16;
  const int half = d / 2;
  const long long total = rows * heads * slices;
  for (long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x; t < total; t += (long long)gridDim.x * blockDim.x) {
    const int sl = (int)(t % slices);
    const long long rh = t / slices;
    const long long row = rh / heads;
    const __nv_bfloat16* base = x + rh * d;
    float a[8], b[8], oa[8], ob[8];
    unpack8(*reinterpret_cast<const uint4*>(base + sl * 8), a);
    unpack8(*reinterpret_cast<const uint4*>(base + half + sl * 8), b);
    const float4* cs = reinterpret_cast<const float4*>(tab + row * half + sl * 8);     // 8 (cos, sin) pairs = 64 bytes
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = cs[i];
      const float s0 = v.y * sign, s1 = v.w * sign;
      oa[2 * i] = a[2 * i] * v.x - b[2 * i] * s0;
      ob[2 * i] = b[2 * i] * v.x + a[2 * i] * s0;
      oa[2 * i + 1] = a[2 * i + 1] * v.z - b[2 * i + 1] * s1;
      ob[2 * i + 1] = b[2 * i + 1] * v.z + a[2 * i + 1] * s1;
    }
    __nv_bfloat16* ob_ = out + rh * d;
    *reinterpret_cast<uint4*>(ob_ + sl * 8) = pack8(oa);
    *reinterpret_cast<uint4*>(ob_ + half + sl * 8) = pack8(ob);
  }
}

extern "C" int dttt_rope_table(const long long* pos, const float* inv_freq, long long rows, int d, void* tab, cudaStream_t s) {
  if (d % 16) return -2;
  const long long total = rows * (d / 2);
  rope_table_kernel<<<grid_for(total, 256, 148 * 16), 256, 0, s>>>(pos, inv_freq, rows, d / 2, (float2*)tab);
  return (int)cudaGetLastError();
}

extern "C" int dttt_rope_apply(const void* x, void* out, const void* tab, long long rows, int heads, int d, float sign,
                               cudaStream_t s) {
  if (d % 16) return -2;
  long long total = rows * heads * (d / 16);
  rope_apply_kernel<<<grid_for(total, 256, 148 * 32), 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, (const float2*)tab,
                                                                  rows, heads, d, sign);
  return (int)cudaGetLastError();
}

extern "C" int dttt_rope(const void* x, void* out, const long long* pos, const float* inv_freq, long long rows, int heads,
                         int d, float sign, cudaStream_t s) {
  if (d % 16) return -2;
  long long total = rows * heads * (d / 16);
  rope_kernel<<<grid_for(total, 256, 148 * 32), 256, 0, s>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)out, pos, inv_freq, rows,
                                                            heads, d, sign);
  return (int)cudaGetLastError();
}

extern "C" int dttt_swiglu_fwd(const void* g, const void* u, void* y, long long n, cudaStream_t s) {
  if (n % 8) return -2;
  swiglu_fwd_kernel<<<grid_for(n / 8, 256, 148 * 32), 256, 0, s>>>((const uint4*)g, (const uint4*)u, (uint4*)y, n / 8);
  return (int)cudaGetLastError();
}

extern "C" int dttt_swiglu_bwd(const void* g, const void* u, const void* dy, void* dg, void* du, long long n, cudaStream_t s) {
  if (n % 8) return -2;
  swiglu_bwd_kernel<<<grid_for(n / 8, 256, 148 * 32), 256, 0, s>>>((const uint4*)g, (const uint4*)u, (const uint4*)dy,
                                                                  (uint4*)dg, (uint4*)du, n / 8);
  return (int)cudaGetLastError();
}

extern "C" int dttt_adamw(float* p, float* m, float* v, const float* g, long long n, float lr, float b1, float b2, float eps,
                          float wd, float bc1, float bc2, float gscale, cudaStream_t s) {
  if (vec_ok(n, p, m, v, g))
    adamw_kernel_v4<<<grid_for(n / 4, 256, 148 * 8), 256, 0, s>>>((float4*)p, (float4*)m, (float4*)v, (const float4*)g, n / 4, lr, b1, b2,
                                                               eps, wd, bc1, bc2, gscale);
  else
    adamw_kernel<<<grid_for(n, 256, 148 * 16), 256, 0, s>>>(p, m, v, g, n, lr, b1, b2, eps, wd, bc1, bc2, gscale);
  return (int)cudaGetLastError();
}

extern "C" int dttt_seq_sumsq(const void* x, float* out, int B, long long n, int is_bf16, cudaStream_t s) {
  dim3 grid(grid_for(n / 4, 256, 148 * 2), B);
  if (vec_ok(n, x) && (is_bf16 ? n % 8 == 0 : true)) {
    if (is_bf16) seq_sumsq_v4<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, out, n);
    else seq_sumsq_v4<float><<<grid, 256, 0, s>>>((const float*)x, out, n);
    return (int)cudaGetLastError();
  }
  if (is_bf16) seq_sumsq_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, out, n);
  else seq_sumsq_kernel<float><<<grid, 256, 0, s>>>((const float*)x, out, n);
  return (int)cudaGetLastError();
}

extern "C" int dttt_seq_axpy(const float* w, const void* g, const float* coef, float* w_new, void* w_lo, int B, long long n,
                             int g_is_bf16, cudaStream_t s) {
  dim3 grid(grid_for(n / 4, 256, 148 * 4), B);
  if (vec_ok(n, w, g, w_new, w_lo) && n % 8 == 0) {
    if (g_is_bf16) seq_axpy_v4<__nv_bfloat16><<<grid, 256, 0, s>>>(w, (const __nv_bfloat16*)g, coef, w_new, (__nv_bfloat16*)w_lo, n);
    else seq_axpy_v4<float><<<grid, 256, 0, s>>>(w, (const float*)g, coef, w_new, (__nv_bfloat16*)w_lo, n);
    return (int)cudaGetLastError();
  }
  if (g_is_bf16) seq_axpy_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(w, (const __nv_bfloat16*)g, coef, w_new, (__nv_bfloat16*)w_lo, n);
  else seq_axpy_kernel<float><<<grid, 256, 0, s>>>(w, (const float*)g, coef, w_new, (__nv_bfloat16*)w_lo, n);
  return (int)cudaGetLastError();
}

extern "C" int dttt_seq_dot(const float* a, const void* g, float* out, int B, long long n, int g_is_bf16, cudaStream_t s) {
  dim3 grid(grid_for(n / 4, 256, 148 * 2), B);
  if (vec_ok(n, a, g) && n % 8 == 0) {
    if (g_is_bf16) seq_dot_v4<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (const __nv_bfloat16*)g, out, n);
    else seq_dot_v4<float><<<grid, 256, 0, s>>>(a, (const float*)g, out, n);
    return (int)cudaGetLastError();
  }
  if (g_is_bf16) seq_dot_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (const __nv_bfloat16*)g, out, n);
  else seq_dot_kernel<float><<<grid, 256, 0, s>>>(a, (const float*)g, out, n);
  return (int)cudaGetLastError();
}

extern "C" int dttt_seq_lincomb(const float* a, const void* g, const float* alpha, const float* beta, void* out, int B, long long n,
                                int g_is_bf16, cudaStream_t s) {
  dim3 grid(grid_for(n / 4, 256, 148 * 4), B);
  if (vec_ok(n, a, g, out) && n % 8 == 0) {
    if (g_is_bf16) seq_lincomb_v4<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (const __nv_bfloat16*)g, alpha, beta, (__nv_bfloat16*)out, n);
    else seq_lincomb_v4<float><<<grid, 256, 0, s>>>(a, (const float*)g, alpha, beta, (float*)out, n);
    return (int)cudaGetLastError();
  }
  if (g_is_bf16) seq_lincomb_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>(a, (const __nv_bfloat16*)g, alpha, beta, (__nv_bfloat16*)out, n);
  else seq_lincomb_kernel<float><<<grid, 256, 0, s>>>(a, (const float*)g, alpha, beta, (float*)out, n);
  return (int)cudaGetLastError();
}
