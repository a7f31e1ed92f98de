// Two small streaming kernels for the transformer-block glue around the FP8 linears:
//
//   cdb_qk_norm_rope       per-head RMSNorm of a projected q or k, rotary embedding, and the write
//                          into the [text; image] joint-attention buffer, in one pass (the kernel is
//                          scatter_heads_kernel of peer_kernels.cu with one destination)
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

// out[b, s, :] = x[b, s, :] + gate[b, :] * y[b, s, :]; rows of y may be strided (a column slice).
__global__ void __launch_bounds__(256)
    gated_residual_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y, int64_t ld_y,
                          const __nv_bfloat16* __restrict__ gate, int64_t ld_gate, __nv_bfloat16* __restrict__ out,
                          int64_t rows, int64_t rows_per_batch, int cols) {
  pdl_launch_dependents();
  pdl_wait_prior();
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

// Two gated residual adds in one launch (blockIdx.y = job): image and text stream of a double-stream block.
struct GatedJob {
  const __nv_bfloat16* x;
  const __nv_bfloat16* y;
  const __nv_bfloat16* gate;
  __nv_bfloat16* out;
  int64_t ld_y, ld_gate, rows, rows_per_batch;
};
struct GatedJobs {
  GatedJob job[2];
};
__global__ void __launch_bounds__(256) gated_residual_pair_kernel(const __grid_constant__ GatedJobs jobs, int cols) {
  pdl_launch_dependents();
  pdl_wait_prior();
  const GatedJob& j = jobs.job[blockIdx.y];
  const int packs = cols >> 3;
  const int64_t total = j.rows * packs;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
    const int64_t row = i / packs;
    const int p = (int)(i - row * packs);
    const int64_t b = row / j.rows_per_batch;
    const uint4 xv = __ldcs(reinterpret_cast<const uint4*>(j.x + row * cols) + p);
    const uint4 yv = __ldcs(reinterpret_cast<const uint4*>(j.y + row * j.ld_y) + p);
    const uint4 gv = __ldg(reinterpret_cast<const uint4*>(j.gate + b * j.ld_gate) + p);
    uint4 o;
    o.x = b2u(__hadd2_rn(u2b(xv.x), __hmul2_rn(u2b(gv.x), u2b(yv.x))));
    o.y = b2u(__hadd2_rn(u2b(xv.y), __hmul2_rn(u2b(gv.y), u2b(yv.y))));
    o.z = b2u(__hadd2_rn(u2b(xv.z), __hmul2_rn(u2b(gv.z), u2b(yv.z))));
    o.w = b2u(__hadd2_rn(u2b(xv.w), __hmul2_rn(u2b(gv.w), u2b(yv.w))));
    __stcs(reinterpret_cast<uint4*>(j.out + row * cols) + p, o);
  }
}

// ---- few-row bf16 product (adaLN modulation projections kept in bf16) ---------------------------------------
// out[m, n] = bf16( sum_k x[m, k] * w[n, k] + bias[n] ), M <= 4 rows: a weight-streaming pass (HBM-bound, N * K * 2
// bytes), a warp per output column, lanes reading 16-byte pieces of the weight row, fp32 accumulation, the few
// activation rows staged in shared memory as fp32.  Every column is computed by one warp in a fixed order, so
// the result of a column does not depend on which slice of the weight matrix a launch is given: this is what
// lets a context-parallel run shard the columns over the ranks and still get the single-GPU bits.
constexpr int BGEMV_THREADS = 256;
constexpr int BGEMV_MAX_M = 4;

template <int TM>
__global__ void __launch_bounds__(BGEMV_THREADS)
    bf16_gemv_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x, const __nv_bfloat16* __restrict__ w,
                     const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int64_t ld_out, int N,
                     int K) {
  pdl_launch_dependents();
  pdl_wait_prior();
  extern __shared__ __align__(16) float s_x[];  // [TM][K]
  for (int i = threadIdx.x; i < TM * K; i += BGEMV_THREADS) {
    const int m = i / K, k = i - m * K;
    s_x[i] = __bfloat162float(x[(int64_t)m * ld_x + k]);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * BGEMV_THREADS + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * BGEMV_THREADS) >> 5;
  const int chunks = K >> 3;  // 16-byte pieces per weight row
  for (int n = warp; n < N; n += nwarps) {
    const uint4* wrow = reinterpret_cast<const uint4*>(w + (int64_t)n * K);
    float acc[TM];
#pragma unroll
    for (int m = 0; m < TM; ++m) acc[m] = 0.f;
    for (int c0 = lane; c0 < chunks; c0 += 32 * 4) {  // four independent loads in flight per lane
      uint4 wv[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 32;
        wv[j] = c < chunks ? __ldcs(wrow + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = c0 + j * 32;
        if (c < chunks) {
          const uint32_t ww[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
#pragma unroll
          for (int m = 0; m < TM; ++m) {
            const float4* xs = reinterpret_cast<const float4*>(s_x + (int64_t)m * K + c * 8);
            const float4 a = xs[0], b = xs[1];
            acc[m] = fmaf(__uint_as_float(ww[0] << 16), a.x, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[0] & 0xffff0000u), a.y, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[1] << 16), a.z, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[1] & 0xffff0000u), a.w, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[2] << 16), b.x, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[2] & 0xffff0000u), b.y, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[3] << 16), b.z, acc[m]);
            acc[m] = fmaf(__uint_as_float(ww[3] & 0xffff0000u), b.w, acc[m]);
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < TM; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
      const float b = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
      for (int m = 0; m < TM; ++m) out[(int64_t)m * ld_out + n] = __float2bfloat16_rn(acc[m] + b);
    }
  }
}

}  // namespace cdb

using namespace cdb;

extern "C" int cdb_bf16_gemv(const void* x, int64_t ld_x, const void* w, const void* bias, void* out, int64_t ld_out,
                             int64_t M, int64_t N, int64_t K, void* stream) {
  if (!x || !w || !out || M < 0 || N <= 0 || K <= 0 || ld_x < K || ld_out < N) return CDB_ERR_BAD_ARGUMENT;
  if (M == 0) return CDB_OK;
  if (M > BGEMV_MAX_M || K % 8 != 0 || !aligned16(w) || N > INT32_MAX || K > INT32_MAX) return CDB_ERR_UNSUPPORTED;
  const size_t smem = (size_t)M * K * sizeof(float);
  if (smem > 48 * 1024) return CDB_ERR_UNSUPPORTED;  // 4 x 3072 fp32 fits; wider inputs need the tile kernels
  const int64_t want = (N + BGEMV_THREADS / 32 - 1) / (BGEMV_THREADS / 32);
  const int64_t cap = (int64_t)sm_count() * 4;
  const dim3 grid((unsigned)(want < cap ? want : cap));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(bias);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(out);
#define CDB_BGEMV(TM) \
  CDB_CUDA_CHECK(launch_pdl(bf16_gemv_kernel<TM>, grid, dim3(BGEMV_THREADS), smem, st, xp, ld_x, wp, bp, op, ld_out, (int)N, (int)K))
  if (M == 1) CDB_BGEMV(1);
  else if (M == 2) CDB_BGEMV(2);
  else if (M == 3) CDB_BGEMV(3);
  else CDB_BGEMV(4);
#undef CDB_BGEMV
  return CDB_OK;
}


extern "C" int cdb_scatter_heads(const void* x, int64_t ld_x, const void* norm_weight, int norm_across_heads,
                                 const void* cos_table, const void* sin_table, int table_row_offset,
                                 void* const* dst_ptrs, int world, int64_t dst_batch_stride, int64_t tokens,
                                 int64_t tokens_per_batch, int64_t dst_row_offset, int heads, int head_dim, float eps,
                                 void* stream);

// Per-head RMSNorm + rotary embedding into a local joint buffer: the head-scatter kernel with a single
// destination (all heads stay on this GPU).
extern "C" int cdb_qk_norm_rope(const void* x, int64_t ld_x, const void* norm_weight, const void* cos_table,
                                const void* sin_table, void* out, int64_t ld_out, int64_t out_batch_stride,
                                int64_t tokens, int64_t tokens_per_batch, int pos_offset, int heads, int head_dim,
                                float eps, void* stream) {
  if (!norm_weight || !out) return CDB_ERR_BAD_ARGUMENT;
  if (ld_out != (int64_t)heads * head_dim) return CDB_ERR_UNSUPPORTED;  // rows of the joint buffer are dense
  void* dst[1] = {out};
  return cdb_scatter_heads(x, ld_x, norm_weight, 0, cos_table, sin_table, pos_offset, dst, 1, out_batch_stride, tokens,
                           tokens_per_batch, pos_offset, heads, head_dim, eps, stream);
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
  CDB_CUDA_CHECK(launch_pdl(gated_residual_kernel, dim3((unsigned)(blocks < cap ? blocks : cap)), dim3(256), 0,
                            static_cast<cudaStream_t>(stream), static_cast<const __nv_bfloat16*>(x),
                            static_cast<const __nv_bfloat16*>(y), ld_y, static_cast<const __nv_bfloat16*>(gate), ld_gate,
                            static_cast<__nv_bfloat16*>(out), rows, rows_per_batch, (int)cols));
  return CDB_OK;
}

extern "C" int cdb_gated_residual_pair(const void* x, const void* y, int64_t ld_y, const void* gate, int64_t ld_gate,
                                       void* out, int64_t rows, int64_t rows_per_batch, const void* x2, const void* y2,
                                       int64_t ld_y2, const void* gate2, int64_t ld_gate2, void* out2, int64_t rows2,
                                       int64_t rows_per_batch2, int64_t cols, void* stream) {
  if (!x || !y || !gate || !out || !x2 || !y2 || !gate2 || !out2 || rows < 0 || rows2 < 0 || rows_per_batch <= 0 ||
      rows_per_batch2 <= 0 || cols <= 0)
    return CDB_ERR_BAD_ARGUMENT;
  if (rows + rows2 == 0) return CDB_OK;
  if (cols % 8 != 0 || ld_y % 8 != 0 || ld_gate % 8 != 0 || ld_y2 % 8 != 0 || ld_gate2 % 8 != 0 || !aligned16(x) ||
      !aligned16(y) || !aligned16(gate) || !aligned16(out) || !aligned16(x2) || !aligned16(y2) || !aligned16(gate2) ||
      !aligned16(out2))
    return CDB_ERR_UNSUPPORTED;
  GatedJobs jobs{};
  jobs.job[0] = GatedJob{static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(y),
                         static_cast<const __nv_bfloat16*>(gate), static_cast<__nv_bfloat16*>(out), ld_y, ld_gate, rows,
                         rows_per_batch};
  jobs.job[1] = GatedJob{static_cast<const __nv_bfloat16*>(x2), static_cast<const __nv_bfloat16*>(y2),
                         static_cast<const __nv_bfloat16*>(gate2), static_cast<__nv_bfloat16*>(out2), ld_y2, ld_gate2,
                         rows2, rows_per_batch2};
  const int64_t big = (rows > rows2 ? rows : rows2) * (cols / 8);
  const int64_t blocks = (big + 255) / 256;
  const int64_t cap = (int64_t)sm_count() * 8;
  const dim3 grid((unsigned)(blocks < cap ? blocks : cap), 2);
  CDB_CUDA_CHECK(launch_pdl(gated_residual_pair_kernel, grid, dim3(256), 0, static_cast<cudaStream_t>(stream), jobs,
                            (int)cols));
  return CDB_OK;
}
