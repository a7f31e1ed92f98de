// Two small streaming kernels for the transformer-block glue around the FP8 linears:
//
//   qk_norm_rope_kernel    per-head RMSNorm of a projected q or k, rotary embedding, and the write
//                          into the [text; image] joint-attention buffer, in one pass
//   gated_residual_kernel  out = x + gate[b, :] * y  (the adaLN-Zero gated residual add)
//
// In eager PyTorch each of these is 3-8 launches of generic broadcasting kernels (about 40 % of a
// FLUX-shape step's kernel time); here they are one read of the operands and one write.  Both are
// HBM-bound.  Rounding points follow the eager bf16 sequence: the normalised value is rounded once,
// then out = round(round(y * cos) + round(rot(y) * sin)); the gated add is round(x + round(g * y)).
#include "common.cuh"

namespace cdb {

__device__ __forceinline__ __nv_bfloat162 u2b(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t b2u(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

// One CTA of QK_THREADS threads per token (grid-stride).  The token's heads*head_dim values are
// 16-byte packets of 8 elements; thread t owns packets t, t + 128, ...  A head is LPH = head_dim/8
// consecutive packets, i.e. LPH consecutive lanes, and because 128 % LPH == 0 every packet of a
// thread sits at the same place inside its head: the thread's slice of the norm weight and of the
// token's cos / sin rows is loaded once and reused for all heads.  Sum of squares per head =
// butterfly over LPH lanes.  All of a thread's packets are requested before any is used.
constexpr int QK_THREADS = 128;
constexpr int QK_PK = 4;  // packets per thread and pass (3 are used for 24 heads x 128)

template <int LPH>
__global__ void __launch_bounds__(QK_THREADS)
    qk_norm_rope_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ cs, const __nv_bfloat16* __restrict__ sn,
                        __nv_bfloat16* __restrict__ out, int64_t ld_out, int64_t out_batch_stride,
                        int64_t tokens, int64_t tokens_per_batch, int pos_offset, int heads, float eps) {
  constexpr int D = LPH * 8;
  const int npk = heads * LPH;
  const int in_head = threadIdx.x % LPH;  // packet index inside the head, the same for all of this thread's packets
  const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + in_head);
  const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
  for (int64_t tok = blockIdx.x; tok < tokens; tok += gridDim.x) {
    const int64_t b = tok / tokens_per_batch, t = tok - b * tokens_per_batch;
    const int64_t pos = (int64_t)pos_offset + t;
    const uint4* src = reinterpret_cast<const uint4*>(x + tok * ld_x);
    uint4* dst = reinterpret_cast<uint4*>(out + b * out_batch_stride + pos * ld_out);
    const uint4 cv = __ldg(reinterpret_cast<const uint4*>(cs + pos * D) + in_head);
    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sn + pos * D) + in_head);
    const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
    for (int base = 0; base < npk; base += QK_THREADS * QK_PK) {
      uint4 v[QK_PK];
#pragma unroll
      for (int j = 0; j < QK_PK; ++j) {
        const int p = base + j * QK_THREADS + threadIdx.x;
        v[j] = p < npk ? __ldcs(src + p) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < QK_PK; ++j) {
        const int p = base + j * QK_THREADS + threadIdx.x;
        const uint32_t xw[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = __uint_as_float(xw[i] << 16), hi = __uint_as_float(xw[i] & 0xffff0000u);
          ss += lo * lo + hi * hi;
        }
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float rstd = rsqrtf(ss / (float)D + eps);
        uint32_t ow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = __uint_as_float(xw[i] << 16), hi = __uint_as_float(xw[i] & 0xffff0000u);
          const float wlo = __uint_as_float(ww[i] << 16), whi = __uint_as_float(ww[i] & 0xffff0000u);
          const __nv_bfloat162 y = __floats2bfloat162_rn(lo * rstd * wlo, hi * rstd * whi);
          // rotation partner of the pair (y0, y1) is (-y1, y0)
          const __nv_bfloat162 r = __halves2bfloat162(__hneg(__high2bfloat16(y)), __low2bfloat16(y));
          ow[i] = b2u(__hadd2_rn(__hmul2_rn(y, u2b(cw[i])), __hmul2_rn(r, u2b(sw[i]))));
        }
        if (p < npk) __stcs(dst + p, make_uint4(ow[0], ow[1], ow[2], ow[3]));
      }
    }
  }
}

// out[b, s, :] = x[b, s, :] + gate[b, :] * y[b, s, :]; rows of y may be strided (a column slice).
__global__ void __launch_bounds__(256)
    gated_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y, int64_t ld_y,
                          const __nv_bfloat16* __restrict__ gate, int64_t ld_gate, __nv_bfloat16* __restrict__ out,
                          int64_t rows, int64_t rows_per_batch, int cols) {
  const int packs = cols >> 3;
  const int64_t total = rows * packs;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / packs;
    const int p = (int)(i - row * packs);
    const int64_t b = row / rows_per_batch;
    const uint4 xv = __ldcs(reinterpret_cast<const uint4*>(x + row * cols) + p);
    const uint4 yv = __ldcs(reinterpret_cast<const uint4*>(y + row * ld_y) + p);
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(gate + b * ld_gate) + p);
    uint4 o;
    o.x = b2u(__hadd2_rn(u2b(xv.x), __hmul2_rn(u2b(gv.x), u2b(yv.x))));
    o.y = b2u(__hadd2_rn(u2b(xv.y), __hmul2_rn(u2b(gv.y), u2b(yv.y))));
    o.z = b2u(__hadd2_rn(u2b(xv.z), __hmul2_rn(u2b(gv.z), u2b(yv.z))));
    o.w = b2u(__hadd2_rn(u2b(xv.w), __hmul2_rn(u2b(gv.w), u2b(yv.w))));
    __stcs(reinterpret_cast<uint4*>(out + row * cols) + p, o);
  }
}

}  // namespace cdb

using namespace cdb;

extern "C" int cdb_qk_norm_rope(const void* x, int64_t ld_x, const void* norm_weight, const void* cos_table,
                                const void* sin_table, void* out, int64_t ld_out, int64_t out_batch_stride,
                                int64_t tokens, int64_t tokens_per_batch, int pos_offset, int heads, int head_dim,
                                float eps, void* stream) {
  if (!x || !norm_weight || !cos_table || !sin_table || !out || tokens < 0 || tokens_per_batch <= 0 || heads <= 0)
    return CDB_ERR_BAD_ARGUMENT;
  if (tokens == 0) return CDB_OK;
  if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || ld_x % 8 != 0 || ld_out % 8 != 0 ||
      out_batch_stride % 8 != 0 || !aligned16(x) || !aligned16(out) || !aligned16(norm_weight) ||
      !aligned16(cos_table) || !aligned16(sin_table))
    return CDB_ERR_UNSUPPORTED;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t cap = (int64_t)sm_count() * 16;  // 16 CTAs of 128 threads per SM: one resident wave
  const unsigned grid = (unsigned)(tokens < cap ? tokens : cap);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(norm_weight);
  const __nv_bfloat16* cp = static_cast<const __nv_bfloat16*>(cos_table);
  const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(sin_table);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
#define CDB_QK(LPH)                                                                                          \
  qk_norm_rope_kernel<LPH><<<grid, QK_THREADS, 0, st>>>(xp, ld_x, wp, cp, sp, op, ld_out, out_batch_stride, \
                                                        tokens, tokens_per_batch, pos_offset, heads, eps)
  if (head_dim == 64) CDB_QK(8);
  else if (head_dim == 128) CDB_QK(16);
  else CDB_QK(32);
#undef CDB_QK
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_gated_residual(const void* x, const void* y, int64_t ld_y, const void* gate, int64_t ld_gate,
                                  void* out, int64_t rows, int64_t rows_per_batch, int64_t cols, void* stream) {
  if (!x || !y || !gate || !out || rows < 0 || rows_per_batch <= 0 || cols <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (rows == 0) return CDB_OK;
  if (cols % 8 != 0 || ld_y % 8 != 0 || ld_gate % 8 != 0 || !aligned16(x) || !aligned16(y) || !aligned16(gate) ||
      !aligned16(out))
    return CDB_ERR_UNSUPPORTED;
  const int64_t total = rows * (cols / 8);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  gated_residual_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y), ld_y,
      static_cast<const __nv_bfloat16*>(gate), ld_gate, static_cast<__nv_bfloat16*>(out), rows, rows_per_batch,
      (int)cols);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}
