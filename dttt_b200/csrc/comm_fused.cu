// Peer-memory plumbing and the fused optimiser-step collectives.
//
// Buffers that other ranks of the node read or write are allocated here with cudaMalloc and exchanged as CUDA
// IPC handles, so a kernel on rank r holds a plain device pointer to every peer's copy and moves data over
// NVLink / NVSwitch with ordinary loads and stores (no library collective in the loop):
//
//   reduce_scatter_sumsq   out[i] = scale * sum_p grad_p[off + i]  for this rank's slice, read from every peer's
//                          full f32 gradient buffer, plus the slice's sum of squares (for the global clip norm):
//                          the FSDP gradient reduce-scatter and the cast/scale pass in one kernel.
//   adamw_allgather        AdamW on this rank's f32 master / moment slices, then the updated parameter is written
//                          in the compute dtype into EVERY rank's compute-copy buffer at [off + i]: the sharded
//                          update and the parameter all-gather in one kernel.
//
// Ordering between ranks is provided by the caller (a stream-ordered barrier before the first kernel, the scalar
// all-reduce of the norm between the two, a barrier after the second); the kernels themselves never wait on a
// peer, so they cannot hang on one.  16-byte vector accesses; n and off are multiples of 8 elements.
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <string.h>

#define DTTT_MAX_PEERS 16

struct PeerPtrs {
  void* p[DTTT_MAX_PEERS];
};

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void reduce_scatter_sumsq_kernel(PeerPtrs peers, int world, int self, long long off, long long n, float scale,
                                            float* __restrict__ out, float* __restrict__ sumsq) {
  float ss = 0.f;
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    // start at this rank's own copy and walk the ring, so concurrent ranks pull from different peers
    for (int k = 0; k < world; ++k) {
      const int p = (self + k) % world;
      const float4 v = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(peers.p[p]) + off)[i];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= scale; acc.y *= scale; acc.z *= scale; acc.w *= scale;
    reinterpret_cast<float4*>(out)[i] = acc;
    ss += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  ss = warp_sum(ss);
  __shared__ float red[32];
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    ss = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    ss = warp_sum(ss);
    if (threadIdx.x == 0 && sumsq) atomicAdd(sumsq, ss);
  }
}

template <bool LO_BF16>
__global__ void adamw_allgather_kernel(float* __restrict__ p, float* __restrict__ m, float* __restrict__ v,
                                       const float* __restrict__ g, long long n, float lr, float b1, float b2, float eps,
                                       float wd, float bc1, float bc2, float gscale, PeerPtrs lo, int world, int self,
                                       long long off) {
  const long long n4 = n / 4;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 gp = reinterpret_cast<const float4*>(g)[i];
    float4 mp = reinterpret_cast<float4*>(m)[i], vp = reinterpret_cast<float4*>(v)[i], pp = reinterpret_cast<float4*>(p)[i];
    float* gg = &gp.x; float* mm = &mp.x; float* vv = &vp.x; float* pw = &pp.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float x = gg[j] * gscale;
      mm[j] = b1 * mm[j] + (1.f - b1) * x;
      vv[j] = b2 * vv[j] + (1.f - b2) * x * x;
      const float upd = (mm[j] / bc1) / (sqrtf(vv[j] / bc2) + eps) + wd * pw[j];
      pw[j] = pw[j] - lr * upd;
    }
    reinterpret_cast<float4*>(m)[i] = mp;
    reinterpret_cast<float4*>(v)[i] = vp;
    reinterpret_cast<float4*>(p)[i] = pp;
    if (LO_BF16) {
      uint2 packed;
      __nv_bfloat162* pb = reinterpret_cast<__nv_bfloat162*>(&packed);
      pb[0] = __floats2bfloat162_rn(pp.x, pp.y);
      pb[1] = __floats2bfloat162_rn(pp.z, pp.w);
      for (int k = 0; k < world; ++k) {
        const int r = (self + k) % world;
        reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(lo.p[r]) + off)[i] = packed;
      }
    } else {
      for (int k = 0; k < world; ++k) {
        const int r = (self + k) % world;
        reinterpret_cast<float4*>(reinterpret_cast<float*>(lo.p[r]) + off)[i] = pp;
      }
    }
  }
  __threadfence_system();
}

inline int grid_for(long long n, int block, int cap) {
  long long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

// ---------------------------------------------------------------- peer memory (CUDA IPC)
extern "C" int dttt_peer_alloc(void** ptr, long long bytes) {
  cudaError_t e = cudaMalloc(ptr, (size_t)bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, (size_t)bytes);
  return (int)e;
}
extern "C" int dttt_peer_free(void* ptr) { return (int)cudaFree(ptr); }
extern "C" int dttt_peer_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e == cudaSuccess) memcpy(handle64, &h, sizeof(h));
  return (int)e;
}
extern "C" int dttt_peer_open(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return (int)cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
}
extern "C" int dttt_peer_close(void* ptr) { return (int)cudaIpcCloseMemHandle(ptr); }
extern "C" int dttt_ipc_handle_bytes() { return (int)sizeof(cudaIpcMemHandle_t); }

// ---------------------------------------------------------------- fused collectives
extern "C" int dttt_reduce_scatter_sumsq(void* const* peer_grads, int world, int self, long long off, long long n, float scale,
                                         float* out, float* sumsq, cudaStream_t s) {
  if (world > DTTT_MAX_PEERS || (n % 4) || (off % 4)) return -2;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = peer_grads[i];
  reduce_scatter_sumsq_kernel<<<grid_for(n / 4, 256, 148 * 8), 256, 0, s>>>(pp, world, self, off, n, scale, out, sumsq);
  return (int)cudaGetLastError();
}

extern "C" int dttt_adamw_allgather(float* p, float* m, float* v, const float* g, long long n, float lr, float b1, float b2,
                                    float eps, float wd, float bc1, float bc2, float gscale, void* const* peer_lo, int world,
                                    int self, long long off, int lo_is_bf16, cudaStream_t s) {
  if (world > DTTT_MAX_PEERS || (n % 4) || (off % 4)) return -2;
  PeerPtrs pp;
  for (int i = 0; i < world; ++i) pp.p[i] = peer_lo[i];
  const int grid = grid_for(n / 4, 256, 148 * 8);
  if (lo_is_bf16)
    adamw_allgather_kernel<true><<<grid, 256, 0, s>>>(p, m, v, g, n, lr, b1, b2, eps, wd, bc1, bc2, gscale, pp, world, self, off);
  else
    adamw_allgather_kernel<false><<<grid, 256, 0, s>>>(p, m, v, g, n, lr, b1, b2, eps, wd, bc1, bc2, gscale, pp, world, self, off);
  return (int)cudaGetLastError();
}
