// Per-row dynamic FP8 (e4m3fn) quantization for sm_100a, optionally fused with the op that
// produces the row (adaLN-modulated LayerNorm, tanh-GELU).
//
// A row is owned by 32, 64, 128 or 256 threads (one warp up to 3072 columns, so the common
// case needs no block barrier) and stays in registers as packed bf16 between the amax pass and
// the conversion pass: every input byte is read from HBM exactly once and only the 1-byte codes
// plus one float per row are written.  HBM-bound: 2 B read + 1 B written per element.
#include <cuda_fp8.h>

#include <cstdint>
#include <cstdlib>

#include "common.cuh"

namespace cdb {

constexpr float E4M3_MAX = 448.0f;

struct QuantFuse {
  const __nv_bfloat16* shift;  // [batch, cols] (row stride ld_mod)
  const __nv_bfloat16* scale;
  int64_t rows_per_batch;
  int64_t ld_mod;
  float eps;
  // CDB_PRE_CONCAT_GELU: the row is [x row | gelu(tail row)]; the first `head_packs` 16-byte
  // packets come from x, the rest from `tail` (row stride ld_tail)
  const __nv_bfloat16* tail;
  int64_t ld_tail;
  int head_packs;
  int tail_plain;  // CDB_PRE_CONCAT_GELU only: the tail already is activated (the product that wrote it did it)
  // Second tensor quantized by the same launch (x2 != nullptr): rows [rows1, rows) of the launch are its
  // rows 0..; it has its own modulation vectors and outputs.  Used for the image and the text stream of a
  // double-stream block, whose text part alone would be a launch of a few microseconds.
  const __nv_bfloat16* x2;
  int64_t rows1, ld_x2;
  const __nv_bfloat16* shift2;
  const __nv_bfloat16* scale2;
  int64_t rows_per_batch2, ld_mod2;
  uint8_t* q2;
  float* scale_out2;
};

// bf16x2 word <-> two floats (bf16 -> fp32 is a 16-bit shift: no conversion instruction)
__device__ __forceinline__ float lo_f(uint32_t u) { return __uint_as_float(u << 16); }
__device__ __forceinline__ float hi_f(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ __nv_bfloat162 as_bf2(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// Four floats -> four e4m3 codes (round to nearest even, saturating) in one word, a in the lowest byte: two
// conversion instructions and one register pairing.
__device__ __forceinline__ uint32_t e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  uint32_t r;
  asm("mov.b32 %0, {%1, %2};" : "=r"(r) : "h"(lo), "h"(hi));
  return r;
}

constexpr int Q_CTA = 256;  // threads per CTA; a CTA works on Q_CTA / TPR rows at once

// Reduction over the TPR threads that share a row: shuffles inside the warp, then (TPR > 32)
// one shared-memory exchange between the row's warps.  `slot` alternates so that one
// barrier per reduction is enough.
template <int TPR, bool MAX>
__device__ __forceinline__ float row_reduce(float v, float (*s_red)[Q_CTA / 32], int& slot) {
  v = MAX ? warp_max(v) : warp_sum(v);
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;  // warps per row
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane == 0) s_red[slot][warp] = v;
    // only the warps of this row wait for each other (named barrier 1 + row group)
    asm volatile("bar.sync %0, %1;" ::"r"(1 + (int)threadIdx.x / TPR), "n"(TPR) : "memory");
    const int first = (warp / WPR) * WPR;
    float r = s_red[slot][first];
#pragma unroll
    for (int w = 1; w < WPR; ++w) r = MAX ? fmaxf(r, s_red[slot][first + w]) : r + s_red[slot][first + w];
    slot = (slot + 1) % 3;
    return r;
  } else {
    return v;
  }
}

// TPR threads per row (a warp for rows up to 3072 columns, so most rows need no barrier at all),
// VPT 16-byte packets per thread kept as packed bf16 in registers between the amax pass and the
// conversion pass.
template <int TPR, int VPT, int PREOP>
__global__ void __launch_bounds__(Q_CTA)
    fp8_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int cols, int64_t ld_x,
                          const QuantFuse f, uint8_t* __restrict__ q, float* __restrict__ scale) {
  constexpr int RPC = Q_CTA / TPR;  // rows per CTA and iteration
  pdl_launch_dependents();
  pdl_wait_prior();
  __shared__ float s_red[3][Q_CTA / 32];
  int slot = 0;
  const int npack = cols >> 3;
  const int group = threadIdx.x / TPR, tig = threadIdx.x % TPR;
  const int64_t iters = (rows + (int64_t)gridDim.x * RPC - 1) / ((int64_t)gridDim.x * RPC);
  // LayerNorm variant: a thread owns the same columns in every row it sees, so its slice of
  // round(1 + scale) and of shift stays in registers until the batch index changes.
  constexpr int MV = PREOP == CDB_PRE_LAYERNORM_MOD ? VPT : 1;
  uint4 m_one_plus[MV], m_shift[MV];
  int64_t m_batch = INT64_MIN;
  // Rows [rows1, rows) belong to the second tensor of a two-tensor launch.
  auto second = [&](int64_t row) { return f.x2 != nullptr && row >= f.rows1; };
  auto row_ptr = [&](int64_t row) -> const __nv_bfloat16* {
    return second(row) ? f.x2 + (row - f.rows1) * f.ld_x2 : x + row * ld_x;
  };
  // One row's packets for this thread; rows past the end and packets past the row load zeros.
  auto load_row = [&](int64_t row, uint4 (&dst)[VPT]) {
    const bool valid = row < rows;
    const __nv_bfloat16* xr = row_ptr(valid ? row : 0);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int p = tig + k * TPR;
      const uint4* src = reinterpret_cast<const uint4*>(xr) + p;
      if constexpr (PREOP == CDB_PRE_CONCAT_GELU) {
        if (p >= f.head_packs)
          src = reinterpret_cast<const uint4*>(f.tail + (valid ? row : 0) * f.ld_tail) + (p - f.head_packs);
      }
      dst[k] = (valid && p < npack) ? __ldcs(src) : make_uint4(0, 0, 0, 0);
    }
  };
  auto row_of = [&](int64_t it) { return (it * gridDim.x + blockIdx.x) * RPC + group; };

  // The next row is requested while the current one is reduced and converted.  The LayerNorm
  // variant (long dependent chain per row, 2 CTAs per SM either way) holds it in registers; the
  // others only pull it into L2, which costs no registers and so keeps 5 CTAs per SM resident.
  constexpr bool REG_PREFETCH = PREOP == CDB_PRE_LAYERNORM_MOD;
  auto prefetch_row_l2 = [&](int64_t row) {
    if (row >= rows) return;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int p = tig + k * TPR;
      const uint4* src = reinterpret_cast<const uint4*>(row_ptr(row)) + p;
      if constexpr (PREOP == CDB_PRE_CONCAT_GELU) {
        if (p >= f.head_packs) src = reinterpret_cast<const uint4*>(f.tail + row * f.ld_tail) + (p - f.head_packs);
      }
      if (p < npack) asm volatile("prefetch.global.L2 [%0];" ::"l"(src));
    }
  };
  uint4 pk[VPT], nxt[REG_PREFETCH ? VPT : 1];
  if constexpr (REG_PREFETCH) load_row(row_of(0), nxt);
  for (int64_t it = 0; it < iters; ++it) {  // same trip count for every thread: barriers stay aligned
    const int64_t row = row_of(it);
    const bool valid = row < rows;
    if constexpr (REG_PREFETCH) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) pk[k] = nxt[k];
      if (it + 1 < iters) load_row(row_of(it + 1), nxt);
    } else {
      load_row(row, pk);
      if (it + 1 < iters) prefetch_row_l2(row_of(it + 1));
    }

    if constexpr (PREOP == CDB_PRE_LAYERNORM_MOD) {
      // LayerNorm statistics in fp32 from registers (two passes over values unpacked once), the
      // normalised value rounded to bf16, then y = round(round(norm * round(1 + scale)) + shift):
      // the rounding points of the eager bf16 modulation, done with packed bf16 arithmetic.
      float xf[VPT][8];
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const uint32_t w[4] = {pk[k].x, pk[k].y, pk[k].z, pk[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xf[k][2 * j] = lo_f(w[j]);
          xf[k][2 * j + 1] = hi_f(w[j]);
          s += xf[k][2 * j] + xf[k][2 * j + 1];
        }
      }
      const float mean = row_reduce<TPR, false>(s, s_red, slot) / (float)cols;
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        if (tig + k * TPR < npack) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            xf[k][j] -= mean;
            ss = fmaf(xf[k][j], xf[k][j], ss);
          }
        }
      }
      const float var = row_reduce<TPR, false>(ss, s_red, slot) / (float)cols;
      const float rstd = rsqrtf(var + f.eps);
      const int64_t vrow = valid ? row : 0;
      const bool sec = second(vrow);
      const int64_t bidx = sec ? (vrow - f.rows1) / f.rows_per_batch2 : vrow / f.rows_per_batch;
      const int64_t mod_key = sec ? ~bidx : bidx;  // distinct keys for the two tensors' batches
      if (mod_key != m_batch) {
        m_batch = mod_key;
        const uint4* sh = reinterpret_cast<const uint4*>(sec ? f.shift2 + bidx * f.ld_mod2 : f.shift + bidx * f.ld_mod);
        const uint4* sc = reinterpret_cast<const uint4*>(sec ? f.scale2 + bidx * f.ld_mod2 : f.scale + bidx * f.ld_mod);
        const __nv_bfloat162 one = __float2bfloat162_rn(1.0f);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int p = tig + k * TPR;
          if (p < npack) {
            const uint4 vsc = __ldg(sc + p);
            m_shift[k] = __ldg(sh + p);
            m_one_plus[k] = make_uint4(as_u32(__hadd2_rn(one, as_bf2(vsc.x))), as_u32(__hadd2_rn(one, as_bf2(vsc.y))),
                                       as_u32(__hadd2_rn(one, as_bf2(vsc.z))), as_u32(__hadd2_rn(one, as_bf2(vsc.w))));
          }
        }
      }
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int p = tig + k * TPR;
        if (p < npack) {
          uint32_t w[4];
          const uint32_t wsh[4] = {m_shift[k].x, m_shift[k].y, m_shift[k].z, m_shift[k].w};
          const uint32_t wop[4] = {m_one_plus[k].x, m_one_plus[k].y, m_one_plus[k].z, m_one_plus[k].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 nrm = as_bf2(pack2(xf[k][2 * j] * rstd, xf[k][2 * j + 1] * rstd));
            w[j] = as_u32(__hadd2_rn(__hmul2_rn(nrm, as_bf2(wop[j])), as_bf2(wsh[j])));
          }
          pk[k] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    } else if constexpr (PREOP == CDB_PRE_GELU_TANH) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        uint32_t w[4] = {pk[k].x, pk[k].y, pk[k].z, pk[k].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) w[j] = pack2(gelu_tanh(lo_f(w[j])), gelu_tanh(hi_f(w[j])));
        pk[k] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    } else if constexpr (PREOP == CDB_PRE_CONCAT_GELU) {
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        if (tig + k * TPR >= f.head_packs && !f.tail_plain) {
          uint32_t w[4] = {pk[k].x, pk[k].y, pk[k].z, pk[k].w};
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = pack2(gelu_tanh(lo_f(w[j])), gelu_tanh(hi_f(w[j])));
          pk[k] = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
    }

    // row maximum of |y| with packed bf16 ops (exact: max and abs do not round)
    __nv_bfloat162 m2 = __float2bfloat162_rn(0.f);
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      m2 = __hmax2(m2, __habs2(as_bf2(pk[k].x)));
      m2 = __hmax2(m2, __habs2(as_bf2(pk[k].y)));
      m2 = __hmax2(m2, __habs2(as_bf2(pk[k].z)));
      m2 = __hmax2(m2, __habs2(as_bf2(pk[k].w)));
    }
    const uint32_t mu = as_u32(m2);
    const float amax = row_reduce<TPR, true>(fmaxf(lo_f(mu), hi_f(mu)), s_red, slot);
    // amax / 448 the way PyTorch's CUDA division by a Python scalar computes it: times fl32(1/448)
    float sc = __fmul_rn(amax, 1.0f / E4M3_MAX);
    if (sc == 0.f) sc = 1.f;  // all-zero row: keep zeros exact instead of 0/0
    const bool out2 = valid && second(row);
    if (valid && tig == 0) {
      if (out2) f.scale_out2[row - f.rows1] = sc;
      else scale[row] = sc;
    }

    // x / sc with one reciprocal per row.  Plain variant (weights, bit-exact against the reference's
    // division): t = x * (1/sc) followed by one Newton correction (r = x - t*sc exactly by FMA;
    // t += r * (1/sc)) reproduces the correctly rounded quotient.  Fused variants: the producer
    // already differs from an eager pipeline in the last bit of a few values per million, and
    // x * (1/sc) can change an e4m3 code only when the quotient is within two fp32 ulps of a rounding
    // midpoint (about 2^-19 of the elements), so the correction is dropped.  Rows whose scale is so
    // small that 1/sc would overflow take the plain division.
    uint8_t* qr = out2 ? f.q2 + (row - f.rows1) * (int64_t)cols : q + (valid ? row : 0) * (int64_t)cols;
    if (sc >= 1e-30f) {  // same for every thread of the row, so the branch is uniform per warp
      const float inv = __frcp_rn(sc);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int p = tig + k * TPR;
        if (valid && p < npack) {
          const uint32_t w[4] = {pk[k].x, pk[k].y, pk[k].z, pk[k].w};
          float t[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float v0 = lo_f(w[j]), v1 = hi_f(w[j]);
            t[2 * j] = v0 * inv;
            t[2 * j + 1] = v1 * inv;
            if constexpr (PREOP == CDB_PRE_NONE) {
              // copysign: the correction of a zero quotient is +0, which would turn -0 into +0
              t[2 * j] = copysignf(fmaf(fmaf(-t[2 * j], sc, v0), inv, t[2 * j]), v0);
              t[2 * j + 1] = copysignf(fmaf(fmaf(-t[2 * j + 1], sc, v1), inv, t[2 * j + 1]), v1);
            }
          }
          __stcs(reinterpret_cast<uint2*>(qr + (int64_t)p * 8),
                 make_uint2(e4m3x4(t[0], t[1], t[2], t[3]), e4m3x4(t[4], t[5], t[6], t[7])));
        }
      }
    } else {  // a scale so small that its reciprocal would overflow: plain division
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int p = tig + k * TPR;
        if (valid && p < npack) {
          const uint32_t w[4] = {pk[k].x, pk[k].y, pk[k].z, pk[k].w};
          __stcs(reinterpret_cast<uint2*>(qr + (int64_t)p * 8),
                 make_uint2(e4m3x4(__fdiv_rn(lo_f(w[0]), sc), __fdiv_rn(hi_f(w[0]), sc), __fdiv_rn(lo_f(w[1]), sc),
                                   __fdiv_rn(hi_f(w[1]), sc)),
                            e4m3x4(__fdiv_rn(lo_f(w[2]), sc), __fdiv_rn(hi_f(w[2]), sc), __fdiv_rn(lo_f(w[3]), sc),
                                   __fdiv_rn(hi_f(w[3]), sc))));
        }
      }
    }
  }
}

template <int TPR, int VPT, int PREOP>
static void launch_quant_variant(const __nv_bfloat16* xp, int64_t rows, int cols, int64_t ld_x, const QuantFuse& f,
                                 uint8_t* qp, float* scale, cudaStream_t st) {
  auto kernel = fp8_quant_rows_kernel<TPR, VPT, PREOP>;
  static PerDevice per_sm_of;
  const int64_t per_sm = per_sm_of.get([&]() -> int64_t {
    int v = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&v, kernel, Q_CTA, 0) != cudaSuccess || v < 1) v = 1;
    return v;
  });
  constexpr int RPC = Q_CTA / TPR;
  const int64_t want = (rows + RPC - 1) / RPC;
  const int64_t wave = (int64_t)per_sm * sm_count();
  const unsigned grid = (unsigned)(want < wave ? want : wave);
  (void)launch_pdl(kernel, dim3(grid), dim3(Q_CTA), 0, st, xp, rows, cols, ld_x, f, qp, scale);
}

template <int PREOP>
static int launch_quant(const void* x, int64_t rows, int64_t cols, int64_t ld_x, const QuantFuse& f,
                        void* q, float* scale, cudaStream_t st) {
  const int npack = (int)(cols / 8);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  uint8_t* qp = static_cast<uint8_t*>(q);
  const int c = (int)cols;
  // Packets per thread: 6 for the plain and GELU variants (measured best on B200: 12 leaves too
  // few rows in flight per SM, 1-4 add barriers without gaining bandwidth), 4 for the LayerNorm
  // variant, which also holds the modulation vectors.  The smallest thread group that fits is
  // used; CDB_QUANT_VMAX overrides the choice for tuning.
  static const int vmax_env = [] { const char* e = getenv("CDB_QUANT_VMAX"); return e ? atoi(e) : 0; }();
  const int vmax = vmax_env > 0 ? vmax_env : (PREOP == CDB_PRE_LAYERNORM_MOD ? 4 : 6);
  int tpr = 32;
  while (tpr < 256 && (npack + tpr - 1) / tpr > vmax) tpr *= 2;
  const int v = (npack + tpr - 1) / tpr;
  if (v > 12) return CDB_ERR_UNSUPPORTED;  // more than 24576 columns
#define CDB_QV(TPR)                                                                              \
  if (v <= 1) launch_quant_variant<TPR, 1, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);         \
  else if (v <= 2) launch_quant_variant<TPR, 2, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);    \
  else if (v <= 3) launch_quant_variant<TPR, 3, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);    \
  else if (v <= 4) launch_quant_variant<TPR, 4, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);    \
  else if (v <= 6) launch_quant_variant<TPR, 6, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);    \
  else if (v <= 8) launch_quant_variant<TPR, 8, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);    \
  else if (v <= 10) launch_quant_variant<TPR, 10, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);  \
  else launch_quant_variant<TPR, 12, PREOP>(xp, rows, c, ld_x, f, qp, scale, st);
  if (tpr == 32) { CDB_QV(32) }
  else if (tpr == 64) { CDB_QV(64) }
  else if (tpr == 128) { CDB_QV(128) }
  else { CDB_QV(256) }
#undef CDB_QV
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

// Two tensors of the same width in one launch (rows of x first, then rows of x2), each with its own
// modulation vectors and outputs.
extern "C" int cdb_fp8_quant_rows_fused_pair(const void* x, int64_t rows, int64_t ld_x, const void* mod_shift,
                                             const void* mod_scale, int64_t rows_per_batch, int64_t ld_mod, void* q,
                                             float* scale, const void* x2, int64_t rows2, int64_t ld_x2,
                                             const void* mod_shift2, const void* mod_scale2, int64_t rows_per_batch2,
                                             int64_t ld_mod2, void* q2, float* scale2, int64_t cols, int preop,
                                             float eps, void* stream) {
  if (!x || !q || !scale || !x2 || !q2 || !scale2 || rows < 0 || rows2 < 0 || cols <= 0 || ld_x < cols || ld_x2 < cols)
    return CDB_ERR_BAD_ARGUMENT;
  if (rows + rows2 == 0) return CDB_OK;
  if (cols % 8 != 0 || ld_x % 8 != 0 || ld_x2 % 8 != 0 || !aligned16(x) || !aligned16(x2) ||
      (reinterpret_cast<uintptr_t>(q) & 7u) || (reinterpret_cast<uintptr_t>(q2) & 7u))
    return CDB_ERR_UNSUPPORTED;
  QuantFuse f{};
  f.x2 = static_cast<const __nv_bfloat16*>(x2);
  f.rows1 = rows;
  f.ld_x2 = ld_x2;
  f.q2 = static_cast<uint8_t*>(q2);
  f.scale_out2 = scale2;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (preop) {
    case CDB_PRE_NONE:
      return launch_quant<CDB_PRE_NONE>(x, rows + rows2, cols, ld_x, f, q, scale, st);
    case CDB_PRE_GELU_TANH:
      return launch_quant<CDB_PRE_GELU_TANH>(x, rows + rows2, cols, ld_x, f, q, scale, st);
    case CDB_PRE_LAYERNORM_MOD:
      if (!mod_shift || !mod_scale || !mod_shift2 || !mod_scale2 || rows_per_batch <= 0 || rows_per_batch2 <= 0 ||
          ld_mod < cols || ld_mod2 < cols)
        return CDB_ERR_BAD_ARGUMENT;
      if (ld_mod % 8 != 0 || ld_mod2 % 8 != 0 || !aligned16(mod_shift) || !aligned16(mod_scale) ||
          !aligned16(mod_shift2) || !aligned16(mod_scale2))
        return CDB_ERR_UNSUPPORTED;
      f.shift = static_cast<const __nv_bfloat16*>(mod_shift);
      f.scale = static_cast<const __nv_bfloat16*>(mod_scale);
      f.rows_per_batch = rows_per_batch;
      f.ld_mod = ld_mod;
      f.shift2 = static_cast<const __nv_bfloat16*>(mod_shift2);
      f.scale2 = static_cast<const __nv_bfloat16*>(mod_scale2);
      f.rows_per_batch2 = rows_per_batch2;
      f.ld_mod2 = ld_mod2;
      f.eps = eps;
      return launch_quant<CDB_PRE_LAYERNORM_MOD>(x, rows + rows2, cols, ld_x, f, q, scale, st);
    default:
      return CDB_ERR_BAD_ARGUMENT;
  }
}

static int quant_rows_concat(const void* head, int64_t head_cols, int64_t ld_head, const void* tail, int64_t tail_cols,
                             int64_t ld_tail, int64_t rows, bool tail_plain, void* q, float* scale, void* stream) {
  if (!head || !tail || !q || !scale || rows < 0 || head_cols <= 0 || tail_cols <= 0 || ld_head < head_cols ||
      ld_tail < tail_cols)
    return CDB_ERR_BAD_ARGUMENT;
  if (rows == 0) return CDB_OK;
  if (head_cols % 8 != 0 || tail_cols % 8 != 0 || ld_head % 8 != 0 || ld_tail % 8 != 0 || !aligned16(head) ||
      !aligned16(tail) || (reinterpret_cast<uintptr_t>(q) & 7u))
    return CDB_ERR_UNSUPPORTED;
  QuantFuse f{};
  f.tail = static_cast<const __nv_bfloat16*>(tail);
  f.ld_tail = ld_tail;
  f.head_packs = (int)(head_cols / 8);
  f.tail_plain = tail_plain ? 1 : 0;
  return launch_quant<CDB_PRE_CONCAT_GELU>(head, rows, head_cols + tail_cols, ld_head, f, q, scale,
                                           static_cast<cudaStream_t>(stream));
}

extern "C" int cdb_fp8_quant_rows_concat_gelu(const void* head, int64_t head_cols, int64_t ld_head,
                                              const void* tail, int64_t tail_cols, int64_t ld_tail, int64_t rows,
                                              void* q, float* scale, void* stream) {
  return quant_rows_concat(head, head_cols, ld_head, tail, tail_cols, ld_tail, rows, false, q, scale, stream);
}

// The same row [head | tail] without the activation: for a tail whose producer already applied it.
extern "C" int cdb_fp8_quant_rows_concat(const void* head, int64_t head_cols, int64_t ld_head, const void* tail,
                                         int64_t tail_cols, int64_t ld_tail, int64_t rows, void* q, float* scale,
                                         void* stream) {
  return quant_rows_concat(head, head_cols, ld_head, tail, tail_cols, ld_tail, rows, true, q, scale, stream);
}

extern "C" int cdb_fp8_quant_rows(const void* x, int64_t rows, int64_t cols, int64_t ld_x, void* q,
                                  float* scale, void* stream) {
  return cdb_fp8_quant_rows_fused(x, rows, cols, ld_x, CDB_PRE_NONE, nullptr, nullptr, 0, 0, 0.f, q,
                                  scale, stream);
}
