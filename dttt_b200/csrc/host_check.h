// Debug checks of what the host hands to the kernels (environment DTTT_DEBUG=1): the memory a tensor map describes, and every
// peer range a fused kernel is given, must lie inside ONE device allocation.  The check is a driver query on the host before
// the launch; a violation is refused with an error code (-70) and nothing is launched.  Off by default: a query per map
// costs about a microsecond per launch.  With torch's caching allocator an "allocation" is the allocator's segment, so the
// check catches extents that leave the segment (wrong strides, counts or offsets), not overlap with a neighbouring tensor.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>

namespace dttt {

inline bool debug_checks_on() {
  static const bool on = [] {
    const char* e = getenv("DTTT_DEBUG");
    return e && e[0] == '1';
  }();
  return on;
}

// 0: [ptr, ptr + bytes) lies inside one allocation, or the range of `ptr` cannot be queried; -70: it does not.
inline int extent_inside_allocation(const void* ptr, unsigned long long bytes) {
  if (!ptr || !bytes) return 0;
  typedef CUresult (*RangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
  static RangeFn fn = [] {
    void* f = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &f, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) f = nullptr;
    return reinterpret_cast<RangeFn>(f);
  }();
  if (!fn) return 0;
  CUdeviceptr base = 0;
  size_t size = 0;
  if (fn(&base, &size, reinterpret_cast<CUdeviceptr>(ptr)) != CUDA_SUCCESS) return 0;
  const unsigned long long lo = reinterpret_cast<unsigned long long>(ptr), hi = lo + bytes;
  return (lo >= base && hi <= base + size) ? 0 : -70;
}

inline int check_extent(const void* ptr, unsigned long long bytes) {
  return debug_checks_on() ? extent_inside_allocation(ptr, bytes) : 0;
}

// Bytes from the base pointer to the end of the last element of a tiled tensor map (dims[0] is the contiguous dimension;
// strides_bytes[i] belongs to dims[i + 1]).
inline unsigned long long map_extent_bytes(int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes, int elem_bytes) {
  unsigned long long e = static_cast<unsigned long long>(dims[0]) * elem_bytes;
  for (int i = 1; i < rank; ++i)
    if (dims[i] > 1) e += static_cast<unsigned long long>(dims[i] - 1) * strides_bytes[i - 1];
  return e;
}

inline int check_map(const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides_bytes, int elem_bytes) {
  if (!debug_checks_on()) return 0;
  if (reinterpret_cast<uintptr_t>(ptr) & 15) return -72;                       // TMA base: 16-byte aligned
  for (int i = 0; i + 1 < rank; ++i)
    if (strides_bytes[i] & 15) return -73;                                     // TMA strides: multiples of 16 bytes
  return extent_inside_allocation(ptr, map_extent_bytes(rank, dims, strides_bytes, elem_bytes));
}

}  // namespace dttt
