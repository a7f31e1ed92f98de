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
// Same slot, free text (used for argument errors that deserve an explanation).
void set_error_text(const char* text);

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

// A value that depends on the device (occupancy, whether a one-time attribute was set), cached per
// device index: function attributes and occupancy belong to the device that is current at the call, so a
// process that drives several GPUs must not reuse what it learnt on the first one.
struct PerDevice {
  static constexpr int kMax = 64;
  int64_t value[kMax] = {};
  bool known[kMax] = {};
  template <class F>
  int64_t get(F&& compute) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMax) return compute();
    if (!known[dev]) {  // concurrent first calls compute the same value twice: harmless
      value[dev] = compute();
      known[dev] = true;
    }
    return value[dev];
  }
};

// Launch with the programmatic-stream-serialization attribute: the kernel's CTAs may be scheduled while the
// previous kernel of the stream is still finishing (once all of ITS blocks have called
// griddepcontrol.launch_dependents or exited), which hides the launch gap between two short kernels.  A kernel
// launched this way must execute griddepcontrol.wait before its first access to global memory.  Works in
// stream capture (the dependency becomes a programmatic edge of the graph).  CDB_PDL=0 turns it off.
bool pdl_enabled();
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                      unsigned cluster_x, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  unsigned n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_x > 1) {  // thread-block clusters of cluster_x CTAs along x (the grid must be a multiple of it)
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
template <class... KArgs, class... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  return launch_pdl_cluster(kernel, grid, block, smem, st, 1u, args...);
}

#ifdef __CUDACC__
// Device side of programmatic dependent launch: let the next kernel of the stream be scheduled while this one
// runs, and wait for the previous kernel (and its memory) before touching global memory.  Both are no-ops for a
// launch without the programmatic-serialization attribute.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait_prior() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
#endif

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- storage-dtype arithmetic policies ------------------------------------------------------
// Every elementwise torch op in the reference materialises its result in the tensor dtype, so
// a chain  c = a - b; d = |c|  is "round after every op".  For 16-bit storage the hardware's
// packed HSUB2/HADD2/HMUL2 (bf16x2 / f16x2) round exactly once to the storage type, which is that
// very semantics (the *_rn forms also forbid contraction into a fused multiply-add) at two
// elements per instruction and without float<->16-bit conversion
// instructions (those issue at a fraction of the FP32 rate and were the limiter of a first
// version that rounded through float).
//
// A policy describes one 32-bit-or-smaller "unit": V = storage of the unit, N = elements in it.
//   sub/add/mul : one rounded op per element        abs      : exact
//   accum       : add every |element| to an fp32 accumulator
//   mulc        : round(c * v) for a float constant c (exact fast path when c is representable)
//   divc        : round(v / w) for a float constant w
struct F32x1 {
  using T = float;
  using V = float;
  static constexpr int N = 1;
  __device__ static __forceinline__ V sub(V a, V b) { return __fsub_rn(a, b); }
  __device__ static __forceinline__ V add(V a, V b) { return __fadd_rn(a, b); }
  __device__ static __forceinline__ V abs(V a) { return fabsf(a); }
  __device__ static __forceinline__ void accum(float& acc, V a) { acc += a; }
  template <bool EXACT>
  __device__ static __forceinline__ V mulc(V a, float c) { return __fmul_rn(c, a); }
  template <bool POW2>
  __device__ static __forceinline__ V divc(V a, float w, float inv_w) {
    return POW2 ? __fmul_rn(a, inv_w) : __fdiv_rn(a, w);
  }
  __device__ static __forceinline__ V zero() { return 0.f; }
  __device__ static __forceinline__ float round1(float v) { return v; }
};

struct BF16x2 {
  using T = __nv_bfloat16;
  using V = __nv_bfloat162;
  static constexpr int N = 2;
  __device__ static __forceinline__ V sub(V a, V b) { return __hsub2_rn(a, b); }
  __device__ static __forceinline__ V add(V a, V b) { return __hadd2_rn(a, b); }
  __device__ static __forceinline__ V abs(V a) { return __habs2(a); }
  __device__ static __forceinline__ void accum(float& acc, V a) {
    const uint32_t u = *reinterpret_cast<uint32_t*>(&a);  // bf16 -> fp32 is a 16-bit shift
    acc += __uint_as_float(u << 16);
    acc += __uint_as_float(u & 0xffff0000u);
  }
  template <bool EXACT>
  __device__ static __forceinline__ V mulc(V a, float c) {
    if constexpr (EXACT) {
      return __hmul2_rn(a, __float2bfloat162_rn(c));
    } else {
      float2 f = __bfloat1622float2(a);
      return __floats2bfloat162_rn(__fmul_rn(c, f.x), __fmul_rn(c, f.y));
    }
  }
  template <bool POW2>
  __device__ static __forceinline__ V divc(V a, float w, float inv_w) {
    if constexpr (POW2) {
      return __hmul2_rn(a, __float2bfloat162_rn(inv_w));
    } else {
      float2 f = __bfloat1622float2(a);
      return __floats2bfloat162_rn(__fdiv_rn(f.x, w), __fdiv_rn(f.y, w));
    }
  }
  __device__ static __forceinline__ V zero() { return __float2bfloat162_rn(0.f); }
  __device__ static __forceinline__ float round1(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

struct BF16x1 {
  using T = __nv_bfloat16;
  using V = __nv_bfloat16;
  static constexpr int N = 1;
  __device__ static __forceinline__ V sub(V a, V b) { return __hsub_rn(a, b); }
  __device__ static __forceinline__ V add(V a, V b) { return __hadd_rn(a, b); }
  __device__ static __forceinline__ V abs(V a) { return __habs(a); }
  __device__ static __forceinline__ void accum(float& acc, V a) { acc += __bfloat162float(a); }
  template <bool EXACT>
  __device__ static __forceinline__ V mulc(V a, float c) {
    return __float2bfloat16_rn(__fmul_rn(c, __bfloat162float(a)));
  }
  template <bool POW2>
  __device__ static __forceinline__ V divc(V a, float w, float) {
    return __float2bfloat16_rn(__fdiv_rn(__bfloat162float(a), w));
  }
  __device__ static __forceinline__ V zero() { return __float2bfloat16_rn(0.f); }
  __device__ static __forceinline__ float round1(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

struct F16x2 {
  using T = __half;
  using V = __half2;
  static constexpr int N = 2;
  __device__ static __forceinline__ V sub(V a, V b) { return __hsub2_rn(a, b); }
  __device__ static __forceinline__ V add(V a, V b) { return __hadd2_rn(a, b); }
  __device__ static __forceinline__ V abs(V a) { return __habs2(a); }
  __device__ static __forceinline__ void accum(float& acc, V a) {
    float2 f = __half22float2(a);
    acc += f.x;
    acc += f.y;
  }
  template <bool EXACT>
  __device__ static __forceinline__ V mulc(V a, float c) {
    if constexpr (EXACT) {
      return __hmul2_rn(a, __float2half2_rn(c));
    } else {
      float2 f = __half22float2(a);
      return __floats2half2_rn(__fmul_rn(c, f.x), __fmul_rn(c, f.y));
    }
  }
  template <bool POW2>
  __device__ static __forceinline__ V divc(V a, float w, float inv_w) {
    // fp16 has a narrow exponent range: a power-of-two scale can still round (subnormals), so
    // always divide in float and round once
    float2 f = __half22float2(a);
    return __floats2half2_rn(__fdiv_rn(f.x, w), __fdiv_rn(f.y, w));
  }
  __device__ static __forceinline__ V zero() { return __float2half2_rn(0.f); }
  __device__ static __forceinline__ float round1(float v) { return __half2float(__float2half_rn(v)); }
};

struct F16x1 {
  using T = __half;
  using V = __half;
  static constexpr int N = 1;
  __device__ static __forceinline__ V sub(V a, V b) { return __hsub_rn(a, b); }
  __device__ static __forceinline__ V add(V a, V b) { return __hadd_rn(a, b); }
  __device__ static __forceinline__ V abs(V a) { return __habs(a); }
  __device__ static __forceinline__ void accum(float& acc, V a) { acc += __half2float(a); }
  template <bool EXACT>
  __device__ static __forceinline__ V mulc(V a, float c) {
    return __float2half_rn(__fmul_rn(c, __half2float(a)));
  }
  template <bool POW2>
  __device__ static __forceinline__ V divc(V a, float w, float) {
    return __float2half_rn(__fdiv_rn(__half2float(a), w));
  }
  __device__ static __forceinline__ V zero() { return __float2half_rn(0.f); }
  __device__ static __forceinline__ float round1(float v) { return __half2float(__float2half_rn(v)); }
};

// 16-byte packet of bf16 for the quantization kernels.
template <typename T>
struct alignas(16) Pack {
  T v[16 / sizeof(T)];
};
template <typename T>
__device__ __forceinline__ Pack<T> ld_stream(const T* p) {
  Pack<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}

// A chunk is U units of policy A handled by one thread at once: U = 16 / sizeof(V) gives one
// streaming 128-bit access (kept out of L1, evict-first in L2), U = 1 with a one-element policy
// is the fallback for pointers that are not 16-byte aligned and for ragged tails.
template <class A, int U>
struct Chunk {
  typename A::V u[U];
};
template <class A, int U>
__device__ __forceinline__ Chunk<A, U> load_chunk(const typename A::T* p) {
  Chunk<A, U> c;
  if constexpr (U * sizeof(typename A::V) == 16) {
    *reinterpret_cast<uint4*>(&c) = __ldcs(reinterpret_cast<const uint4*>(p));
  } else {
    static_assert(U == 1 && A::N == 1, "scalar fallback handles one element");
    c.u[0] = *p;
  }
  return c;
}
template <class A, int U>
__device__ __forceinline__ void store_chunk(typename A::T* p, const Chunk<A, U>& c) {
  if constexpr (U * sizeof(typename A::V) == 16) {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&c));
  } else {
    *p = c.u[0];
  }
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

// tanh-GELU as x * sigmoid(2u), u = sqrt(2/pi) (x + 0.044715 x^3) = x / (1 + 2^(c x (1 + 0.044715 x^2))),
// c = -2 sqrt(2/pi) log2(e): three multiply-adds, one ex2 and one fast division instead of the
// ~25-instruction tanhf (the special-function unit is what bounds this kernel).  The ~1e-6 relative
// error disappears in the rounding of the result to bf16 except for a handful of values per million
// that sit on a rounding boundary.
__device__ __forceinline__ float gelu_tanh(float x) {
  constexpr float c = -2.0f * 0.7978845608028654f * 1.4426950408889634f;
  const float p = fmaf(x * x, c * 0.044715f, c);
  float e;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * p));
  return __fdividef(x, 1.0f + e);
}

}  // namespace cdb
