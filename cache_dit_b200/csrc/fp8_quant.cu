// Per-row dynamic FP8 (e4m3fn) quantization for sm_100a, optionally fused with the op that
// produces the row (adaLN-modulated LayerNorm, tanh-GELU).
//
// One CTA owns one row at a time and keeps the whole row in registers between the amax pass
// and the conversion pass, so every input byte is read from HBM exactly once and only the
// 1-byte codes plus one float per row are written.  HBM-bound: 2 B read + 1 B written per
// element.
#include <cuda_fp8.h>

#include "common.cuh"

namespace cdb {

constexpr int Q_MAX_THREADS = 256;
constexpr int Q_MAX_VPT = 8;            // 16-byte packets per thread -> cols <= 256*8*8 = 16384
constexpr float E4M3_MAX = 448.0f;

struct QuantFuse {
  const __nv_bfloat16* shift;  // [batch, cols] (row stride ld_mod)
  const __nv_bfloat16* scale;
  int64_t rows_per_batch;
  int64_t ld_mod;
  float eps;
};

__device__ __forceinline__ float bf16r(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// Block-wide reductions over <= 8 warps; result broadcast to every thread.
template <bool MAX>
__device__ __forceinline__ float block_reduce(float v, float* smem /*[8]*/) {
  v = MAX ? warp_max(v) : warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  __syncthreads();  // smem may still be read by the previous reduction
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  float r = lane < nwarp ? smem[lane] : (MAX ? 0.f : 0.f);
  r = MAX ? warp_max(r) : warp_sum(r);
  return r;
}

__device__ __forceinline__ float gelu_tanh(float x) {
  const float k0 = 0.7978845608028654f, k1 = 0.044715f;
  float inner = k0 * (x + k1 * x * x * x);
  return 0.5f * x * (1.0f + tanhf(inner));
}

template <int VPT, int PREOP>
__global__ void __launch_bounds__(Q_MAX_THREADS)
    fp8_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int cols, int64_t ld_x,
                          const QuantFuse f, uint8_t* __restrict__ q, float* __restrict__ scale) {
  __shared__ float s_red[8];
  const int npack = cols >> 3;
  for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * ld_x;
    float v[VPT][8];
    bool live[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int p = threadIdx.x + k * blockDim.x;
      live[k] = p < npack;
      if (live[k]) {
        Pack<__nv_bfloat16> pk = ld_stream(xr + (int64_t)p * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = __bfloat162float(pk.v[i]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = 0.f;
      }
    }

    if constexpr (PREOP == CDB_PRE_LAYERNORM_MOD) {
      // LayerNorm statistics in fp32 from registers (two-pass), result rounded to bf16, then
      // y = round(round(norm * round(1 + scale)) + shift) like the eager bf16 modulation.
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k)
#pragma unroll
        for (int i = 0; i < 8; ++i) s += v[k][i];
      const float mean = block_reduce<false>(s, s_red) / (float)cols;
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k)
        if (live[k])
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float d = v[k][i] - mean;
            ss += d * d;
          }
      const float var = block_reduce<false>(ss, s_red) / (float)cols;
      const float rstd = rsqrtf(var + f.eps);
      const int64_t b = row / f.rows_per_batch;
      const __nv_bfloat16* sh = f.shift + b * f.ld_mod;
      const __nv_bfloat16* sc = f.scale + b * f.ld_mod;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        if (!live[k]) continue;
        const int p = threadIdx.x + k * blockDim.x;
        Pack<__nv_bfloat16> psh = *reinterpret_cast<const Pack<__nv_bfloat16>*>(sh + p * 8);
        Pack<__nv_bfloat16> psc = *reinterpret_cast<const Pack<__nv_bfloat16>*>(sc + p * 8);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float nrm = bf16r((v[k][i] - mean) * rstd);
          float one_plus = bf16r(1.0f + __bfloat162float(psc.v[i]));
          v[k][i] = bf16r(bf16r(nrm * one_plus) + __bfloat162float(psh.v[i]));
        }
      }
    } else if constexpr (PREOP == CDB_PRE_GELU_TANH) {
#pragma unroll
      for (int k = 0; k < VPT; ++k)
#pragma unroll
        for (int i = 0; i < 8; ++i) v[k][i] = bf16r(gelu_tanh(v[k][i]));
    }

    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[k][i]));
    amax = block_reduce<true>(amax, s_red);
    float sc = __fdiv_rn(amax, E4M3_MAX);
    if (sc == 0.f) sc = 1.f;  // all-zero row: keep zeros exact instead of 0/0
    if (threadIdx.x == 0) scale[row] = sc;

    // x / sc with one reciprocal per row: t = x * (1/sc) followed by one Newton correction
    // (r = x - t*sc exactly by FMA; t += r * (1/sc)) reproduces the correctly rounded quotient;
    // rows whose scale is so small that 1/sc would overflow take the plain division.
    const bool tiny = sc < 1e-30f;
    const float inv = tiny ? 0.f : __frcp_rn(sc);
    auto quot = [&](float x) -> float {
      if (tiny) return __fdiv_rn(x, sc);
      float t = x * inv;
      float r = fmaf(-t, sc, x);
      return fmaf(r, inv, t);
    };
    uint8_t* qr = q + row * (int64_t)cols;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      if (!live[k]) continue;
      const int p = threadIdx.x + k * blockDim.x;
      uint32_t w[2];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        float2 lo = make_float2(quot(v[k][h * 4 + 0]), quot(v[k][h * 4 + 1]));
        float2 hi = make_float2(quot(v[k][h * 4 + 2]), quot(v[k][h * 4 + 3]));
        uint32_t a = __nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3);
        uint32_t b = __nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3);
        w[h] = a | (b << 16);
      }
      __stcs(reinterpret_cast<uint2*>(qr + (int64_t)p * 8), make_uint2(w[0], w[1]));
    }
  }
}

template <int PREOP>
static int launch_quant(const void* x, int64_t rows, int64_t cols, int64_t ld_x, const QuantFuse& f,
                        void* q, float* scale, cudaStream_t st) {
  const int npack = (int)(cols / 8);
  const int vpt = (npack + Q_MAX_THREADS - 1) / Q_MAX_THREADS;
  if (vpt > Q_MAX_VPT) return CDB_ERR_UNSUPPORTED;
  int threads = (npack + vpt - 1) / vpt;
  threads = (threads + 31) / 32 * 32;
  int64_t cap = (int64_t)sm_count() * (2048 / threads > 16 ? 16 : 2048 / threads);
  const unsigned grid = (unsigned)(rows < cap ? rows : cap);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
#define CDB_Q(V)                                                                                   \
  case V:                                                                                          \
    fp8_quant_rows_kernel<V, PREOP><<<grid, threads, 0, st>>>(xp, rows, (int)cols, ld_x, f, qp, scale); \
    break;
  switch (vpt) {
    CDB_Q(1) CDB_Q(2) CDB_Q(3) CDB_Q(4) CDB_Q(5) CDB_Q(6) CDB_Q(7) CDB_Q(8)
    default: return CDB_ERR_UNSUPPORTED;
  }
#undef CDB_Q
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

}  // namespace cdb

using namespace cdb;

extern "C" int cdb_fp8_quant_rows_fused(const void* x, int64_t rows, int64_t cols, int64_t ld_x,
                                        int preop, const void* mod_shift, const void* mod_scale,
                                        int64_t rows_per_batch, int64_t ld_mod, float eps, void* q,
                                        float* scale, void* stream) {
  if (!x || !q || !scale || rows < 0 || cols <= 0 || ld_x < cols) return CDB_ERR_BAD_ARGUMENT;
  if (rows == 0) return CDB_OK;
  if (cols % 8 != 0 || ld_x % 8 != 0 || !aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u))
    return CDB_ERR_UNSUPPORTED;
  QuantFuse f{};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (preop) {
    case CDB_PRE_NONE:
      return launch_quant<CDB_PRE_NONE>(x, rows, cols, ld_x, f, q, scale, st);
    case CDB_PRE_GELU_TANH:
      return launch_quant<CDB_PRE_GELU_TANH>(x, rows, cols, ld_x, f, q, scale, st);
    case CDB_PRE_LAYERNORM_MOD:
      if (!mod_shift || !mod_scale || rows_per_batch <= 0 || ld_mod < cols) return CDB_ERR_BAD_ARGUMENT;
      if (ld_mod % 8 != 0 || !aligned16(mod_shift) || !aligned16(mod_scale)) return CDB_ERR_UNSUPPORTED;
      f.shift = static_cast<const __nv_bfloat16*>(mod_shift);
      f.scale = static_cast<const __nv_bfloat16*>(mod_scale);
      f.rows_per_batch = rows_per_batch;
      f.ld_mod = ld_mod;
      f.eps = eps;
      return launch_quant<CDB_PRE_LAYERNORM_MOD>(x, rows, cols, ld_x, f, q, scale, st);
    default:
      return CDB_ERR_BAD_ARGUMENT;
  }
}

extern "C" int cdb_fp8_quant_rows(const void* x, int64_t rows, int64_t cols, int64_t ld_x, void* q,
                                  float* scale, void* stream) {
  return cdb_fp8_quant_rows_fused(x, rows, cols, ld_x, CDB_PRE_NONE, nullptr, nullptr, 0, 0, 0.f, q,
                                  scale, stream);
}
