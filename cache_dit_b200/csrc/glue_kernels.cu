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

}  // namespace cdb

using namespace cdb;

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
