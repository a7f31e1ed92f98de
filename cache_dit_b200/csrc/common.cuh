// Shared helpers for the sm_100a kernels: status plumbing, dtype traits, 128-bit access.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/cache_dit_b200.h"

namespace cdb {

// Thread-local text of the last CUDA error; exposed through cdb_last_cuda_error().
void set_cuda_error(cudaError_t e, const char* where);

#define CDB_CUDA_CHECK(expr)                         \
  do {                                               \
    cudaError_t _e = (expr);                         \
    if (_e != cudaSuccess) {                         \
      ::cdb::set_cuda_error(_e, #expr);              \
      return CDB_ERR_CUDA;                           \
    }                                                \
  } while (0)

// Number of SMs of the current device (cached per device).
int sm_count();

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- storage-dtype traits -------------------------------------------------------------
// `round` returns the float nearest-even-rounded to the storage type, as a float: every
// elementwise torch op in the reference materialises its result in the tensor dtype.
template <typename T>
struct DT;

template <>
struct DT<float> {
  static constexpr int VEC = 4;  // elements per 16 bytes
  __device__ static __forceinline__ float load(float v) { return v; }
  __device__ static __forceinline__ float store(float v) { return v; }
  __device__ static __forceinline__ float round(float v) { return v; }
};
template <>
struct DT<__nv_bfloat16> {
  static constexpr int VEC = 8;
  __device__ static __forceinline__ float load(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __forceinline__ __nv_bfloat16 store(float v) { return __float2bfloat16_rn(v); }
  __device__ static __forceinline__ float round(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
  }
};
template <>
struct DT<__half> {
  static constexpr int VEC = 8;
  __device__ static __forceinline__ float load(__half v) { return __half2float(v); }
  __device__ static __forceinline__ __half store(float v) { return __float2half_rn(v); }
  __device__ static __forceinline__ float round(float v) { return __half2float(__float2half_rn(v)); }
};

// 16-byte packet of T.
template <typename T>
struct alignas(16) Pack {
  T v[DT<T>::VEC];
};

// Streaming (read-once / write-once) 128-bit accesses: keep them out of L1 and mark them
// evict-first so the step's tensors do not push the weights out of L2.
template <typename T>
__device__ __forceinline__ Pack<T> ld_stream(const T* p) {
  Pack<T> r;
  uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
  *reinterpret_cast<uint4*>(&r) = u;
  return r;
}
template <typename T>
__device__ __forceinline__ void st_stream(T* p, const Pack<T>& v) {
  __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

}  // namespace cdb
