// Ulysses head/sequence exchange around attention as plain stores into peer GPUs' memory over
// NVLink, fused with the op that produces the data, instead of NCCL all-to-all calls.
//
// Before attention every rank holds q, k, v for ITS tokens and ALL heads; attention wants ALL tokens
// for the rank's OWN heads.  The reference does this with four all-to-all collectives per block
// (src/cache_dit/distributed/transformers/flux.py via diffusers' context-parallel hooks).  Here
//   * scatter_heads_kernel normalises / rotates q and k (or copies v) and writes each head straight
//     into the joint [batch, all tokens, own heads, head_dim] buffer of the rank that owns the head;
//   * gather_tokens_kernel writes each token row of the attention output into the
//     [batch, own tokens, all heads, head_dim] buffer of the rank that owns the token;
//   * peer_signal / peer_wait order the two phases with one flag word per (rank, peer) pair.
// All remote accesses are stores (peer pointers obtained through CUDA IPC by the host side); all
// loads are local: ordinary 16-byte st.global to a mapped peer address, nothing else crosses NVLink.
// Every launch is a fixed sequence of pointers and sizes, so whole block segments, exchange included,
// can be captured in a CUDA graph; the barrier's epoch lives in device memory for that reason.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <cstring>

#include "common.cuh"

namespace cdb {

constexpr int PEER_MAX = 8;

struct PeerPtrs {
  void* p[PEER_MAX];
};

__device__ __forceinline__ __nv_bfloat162 pu2b(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t pb2u(__nv_bfloat162 v) { return *reinterpret_cast<uint32_t*>(&v); }

constexpr int SC_THREADS = 128;
constexpr int SC_PK = 4;

// One CTA per token (grid-stride).  Packets of 8 elements; LPH = head_dim / 8 packets per head.
// Head h goes to rank h / heads_per_rank, as local head h % heads_per_rank, at joint row
// dst_row_offset + (token index inside its batch).
//   MODE 0  copy (the v projection)
//   MODE 1  RMSNorm over each head (weight [head_dim]) + rotary embedding   (FLUX, Qwen-Image)
//   MODE 2  RMSNorm over the whole row (weight [heads * head_dim]) + rotary embedding   (Wan)
constexpr int SCATTER_COPY = 0, SCATTER_HEAD_NORM = 1, SCATTER_ROW_NORM = 2;
template <int LPH, int MODE>
__device__ __forceinline__ void scatter_heads_body(const __nv_bfloat16* __restrict__ x, int64_t ld_x,
                                                   const __nv_bfloat16* __restrict__ w, const __nv_bfloat16* __restrict__ cs,
                                                   const __nv_bfloat16* __restrict__ sn, int table_row_offset,
                                                   const PeerPtrs& dst, int heads_per_rank, int64_t ld_out,
                                                   int64_t out_batch_stride, int64_t tokens, int64_t tokens_per_batch,
                                                   int64_t dst_row_offset, int heads, float eps, float* s_part,
                                                   const PeerPtrs* dst_scale = nullptr) {
  constexpr int D = LPH * 8;
  constexpr bool NORM_ROPE = MODE != SCATTER_COPY;
  const int npk = heads * LPH;
  const int in_head = threadIdx.x % LPH;
  uint32_t ww[4] = {0, 0, 0, 0};
  if constexpr (MODE == SCATTER_HEAD_NORM) {
    const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + in_head);
    ww[0] = wv.x; ww[1] = wv.y; ww[2] = wv.z; ww[3] = wv.w;
  }
  for (int64_t tok = blockIdx.x; tok < tokens; tok += gridDim.x) {
    const int64_t b = tok / tokens_per_batch, t = tok - b * tokens_per_batch;
    const uint4* src = reinterpret_cast<const uint4*>(x + tok * ld_x);
    const int64_t dst_elem = b * out_batch_stride + (dst_row_offset + t) * ld_out;
    uint32_t cw[4] = {0, 0, 0, 0}, sw[4] = {0, 0, 0, 0};
    if constexpr (NORM_ROPE) {
      const int64_t pos = (int64_t)table_row_offset + t;
      const uint4 cv = __ldg(reinterpret_cast<const uint4*>(cs + pos * D) + in_head);
      const uint4 sv = __ldg(reinterpret_cast<const uint4*>(sn + pos * D) + in_head);
      cw[0] = cv.x; cw[1] = cv.y; cw[2] = cv.z; cw[3] = cv.w;
      sw[0] = sv.x; sw[1] = sv.y; sw[2] = sv.z; sw[3] = sv.w;
    }
    float rstd_row = 0.f;
    if constexpr (MODE == SCATTER_ROW_NORM) {  // statistic of the whole row first (the row is re-read from L2 below)
      float ss = 0.f;
      for (int p = threadIdx.x; p < npk; p += SC_THREADS) {
        const uint4 q = __ldg(src + p);
        const uint32_t qw[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float lo = __uint_as_float(qw[i] << 16), hi = __uint_as_float(qw[i] & 0xffff0000u);
          ss += lo * lo + hi * hi;
        }
      }
      ss = warp_sum(ss);
      __syncthreads();  // the previous token's readers of s_part are done
      if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = ss;
      __syncthreads();
      float tot = 0.f;
#pragma unroll
      for (int i = 0; i < SC_THREADS / 32; ++i) tot += s_part[i];
      rstd_row = rsqrtf(tot / (float)(heads * D) + eps);
    }
    for (int base = 0; base < npk; base += SC_THREADS * SC_PK) {
      uint4 v[SC_PK];
#pragma unroll
      for (int j = 0; j < SC_PK; ++j) {
        const int p = base + j * SC_THREADS + threadIdx.x;
        v[j] = p < npk ? __ldcs(src + p) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int j = 0; j < SC_PK; ++j) {
        const int p = base + j * SC_THREADS + threadIdx.x;
        uint32_t ow[4] = {v[j].x, v[j].y, v[j].z, v[j].w};
        if constexpr (NORM_ROPE) {
          float rstd = rstd_row;
          if constexpr (MODE == SCATTER_HEAD_NORM) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float lo = __uint_as_float(ow[i] << 16), hi = __uint_as_float(ow[i] & 0xffff0000u);
              ss += lo * lo + hi * hi;
            }
#pragma unroll
            for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            rstd = rsqrtf(ss / (float)D + eps);
          } else if (p < npk) {  // row norm: the weight differs per packet
            const uint4 wv = __ldg(reinterpret_cast<const uint4*>(w) + p);
            ww[0] = wv.x; ww[1] = wv.y; ww[2] = wv.z; ww[3] = wv.w;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float lo = __uint_as_float(ow[i] << 16), hi = __uint_as_float(ow[i] & 0xffff0000u);
            const float wlo = __uint_as_float(ww[i] << 16), whi = __uint_as_float(ww[i] & 0xffff0000u);
            const __nv_bfloat162 y = __floats2bfloat162_rn(lo * rstd * wlo, hi * rstd * whi);
            const __nv_bfloat162 r = __halves2bfloat162(__hneg(__high2bfloat16(y)), __low2bfloat16(y));
            ow[i] = pb2u(__hadd2_rn(__hmul2_rn(y, pu2b(cw[i])), __hmul2_rn(r, pu2b(sw[i]))));
          }
        }
        if (dst_scale != nullptr) {
          // FP8 on the wire (the reference's `ulysses_float8`, kernels/triton/_float8_comm.py:78-124): one scale
          // per (token, head), s = max(amax / 448, 1e-6), e4m3(clamp(x / s)); the destination holds bytes + scales.
          __nv_bfloat162 m2 = __habs2(pu2b(ow[0]));
#pragma unroll
          for (int i = 1; i < 4; ++i) m2 = __hmax2(m2, __habs2(pu2b(ow[i])));
          const uint32_t mu = pb2u(m2);
          float amax = fmaxf(__uint_as_float(mu << 16), __uint_as_float(mu & 0xffff0000u));
#pragma unroll
          for (int o = LPH / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
          const float sc = fmaxf(__fdiv_rn(amax, 448.0f), 1e-6f);
          // x / sc as one reciprocal per head and a Newton correction per element (t = x * inv; r = x - t * sc
          // exactly by FMA; t + r * inv): the correctly rounded quotient at a third of the instructions of eight
          // IEEE divisions per packet, which made this path issue-bound.  sc >= 1e-6, so 1 / sc cannot overflow.
          const float inv = __frcp_rn(sc);
          auto quot = [&](float v) -> float {
            const float t = v * inv;
            return fmaf(fmaf(-t, sc, v), inv, t);
          };
          if (p < npk) {
            uint32_t q[2];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint32_t a = ow[2 * h], b2 = ow[2 * h + 1];
              const uint32_t lo = __nv_cvt_float2_to_fp8x2(
                  make_float2(quot(__uint_as_float(a << 16)), quot(__uint_as_float(a & 0xffff0000u))),
                  __NV_SATFINITE, __NV_E4M3);
              const uint32_t hi = __nv_cvt_float2_to_fp8x2(
                  make_float2(quot(__uint_as_float(b2 << 16)), quot(__uint_as_float(b2 & 0xffff0000u))),
                  __NV_SATFINITE, __NV_E4M3);
              q[h] = lo | (hi << 16);
            }
            const int head = p / LPH;
            const int owner = head / heads_per_rank;
            const int local_head = head - owner * heads_per_rank;
            uint8_t* base8 = static_cast<uint8_t*>(dst.p[owner]);
            *reinterpret_cast<uint2*>(base8 + dst_elem + (int64_t)local_head * D + (int64_t)(p - head * LPH) * 8) =
                make_uint2(q[0], q[1]);
            if (p == head * LPH)
              static_cast<float*>(dst_scale->p[owner])[dst_elem / D + local_head] = sc;
          }
        } else if (p < npk) {
          const int head = p / LPH;
          const int owner = head / heads_per_rank;
          const int local_head = head - owner * heads_per_rank;
          __nv_bfloat16* base_ptr = static_cast<__nv_bfloat16*>(dst.p[owner]);
          uint4* out = reinterpret_cast<uint4*>(base_ptr + dst_elem + (int64_t)local_head * D) + (p - head * LPH);
          *out = make_uint4(ow[0], ow[1], ow[2], ow[3]);
        }
      }
    }
  }
}

template <int LPH, int MODE>
__global__ void __launch_bounds__(SC_THREADS)
    scatter_heads_kernel(const __nv_bfloat16* __restrict__ x, int64_t ld_x, const __nv_bfloat16* __restrict__ w,
                         const __nv_bfloat16* __restrict__ cs, const __nv_bfloat16* __restrict__ sn, int table_row_offset,
                         const PeerPtrs dst, int heads_per_rank, int64_t ld_out, int64_t out_batch_stride,
                         int64_t tokens, int64_t tokens_per_batch, int64_t dst_row_offset, int heads, float eps) {
  __shared__ float s_part[SC_THREADS / 32];
  scatter_heads_body<LPH, MODE>(x, ld_x, w, cs, sn, table_row_offset, dst, heads_per_rank, ld_out, out_batch_stride,
                                tokens, tokens_per_batch, dst_row_offset, heads, eps, s_part);
}

// Several scatter jobs in one launch (blockIdx.y = job): the q, k and v projections of the text and the
// image stream of one block are up to six jobs, and at small per-rank token counts their launch cost
// exceeded their run time.
constexpr int SCATTER_MAX_JOBS = 6;
struct ScatterJob {
  const __nv_bfloat16* x;
  const __nv_bfloat16* w;
  const __nv_bfloat16* cs;
  const __nv_bfloat16* sn;
  PeerPtrs dst;
  PeerPtrs dst_scale;  // used when fp8_out != 0
  int64_t ld_x, out_batch_stride, tokens, tokens_per_batch, dst_row_offset;
  int table_row_offset, mode, fp8_out;
  float eps;
};
struct ScatterJobs {
  ScatterJob job[SCATTER_MAX_JOBS];
};

template <int LPH>
__global__ void __launch_bounds__(SC_THREADS)
    scatter_heads_multi_kernel(const __grid_constant__ ScatterJobs jobs, int heads_per_rank, int64_t ld_out, int heads) {
  __shared__ float s_part[SC_THREADS / 32];
  const ScatterJob& j = jobs.job[blockIdx.y];
  if ((int64_t)blockIdx.x >= j.tokens) return;
  const PeerPtrs* ds = j.fp8_out ? &j.dst_scale : nullptr;
  if (j.mode == SCATTER_COPY)
    scatter_heads_body<LPH, SCATTER_COPY>(j.x, j.ld_x, j.w, j.cs, j.sn, j.table_row_offset, j.dst, heads_per_rank, ld_out,
                                          j.out_batch_stride, j.tokens, j.tokens_per_batch, j.dst_row_offset, heads,
                                          j.eps, s_part, ds);
  else if (j.mode == SCATTER_HEAD_NORM)
    scatter_heads_body<LPH, SCATTER_HEAD_NORM>(j.x, j.ld_x, j.w, j.cs, j.sn, j.table_row_offset, j.dst, heads_per_rank,
                                               ld_out, j.out_batch_stride, j.tokens, j.tokens_per_batch,
                                               j.dst_row_offset, heads, j.eps, s_part, ds);
  else
    scatter_heads_body<LPH, SCATTER_ROW_NORM>(j.x, j.ld_x, j.w, j.cs, j.sn, j.table_row_offset, j.dst, heads_per_rank,
                                              ld_out, j.out_batch_stride, j.tokens, j.tokens_per_batch,
                                              j.dst_row_offset, heads, j.eps, s_part, ds);
}

// Attention output of this rank, [batch, all tokens, own heads, head_dim]: the row of token s goes
// to the rank whose token range [row_start[r], row_start[r+1]) holds s, into its
// [batch, token capacity, all heads, head_dim] buffer at head offset my_rank * heads_per_rank.
// Ranges may differ in length (token counts that do not divide by the number of ranks).
// One CTA per (batch, token) row, 16-byte packets.
struct PeerRows {
  int64_t start[PEER_MAX + 1];
};

constexpr int GT_UNROLL = 4;
__global__ void __launch_bounds__(256)
    gather_tokens_kernel(const __nv_bfloat16* __restrict__ o, const PeerPtrs dst, const PeerRows rows_of, int world,
                         int my_rank, int64_t batch, int64_t tokens_all, int64_t dst_token_capacity,
                         int heads_per_rank, int heads_all, int head_dim) {
  // Flat over (row, packet): with few heads per rank a row is short (3 heads x 128 = 48 packets), so a CTA per
  // row would leave most of its threads idle; here every thread has GT_UNROLL independent 16-byte copies in flight.
  const int row_packets = heads_per_rank * head_dim / 8;
  const int64_t total = batch * tokens_all * row_packets;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  const uint4* src = reinterpret_cast<const uint4*>(o);
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += GT_UNROLL * stride) {
    uint4 v[GT_UNROLL];
#pragma unroll
    for (int u = 0; u < GT_UNROLL; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) v[u] = __ldcs(src + i);
    }
#pragma unroll
    for (int u = 0; u < GT_UNROLL; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= total) continue;
      const int64_t r = i / row_packets;
      const int p = (int)(i - r * row_packets);
      const int64_t b = r / tokens_all, s = r - b * tokens_all;
      int owner = 0;
      while (owner + 1 < world && s >= rows_of.start[owner + 1]) ++owner;
      const int64_t local_s = s - rows_of.start[owner];
      __nv_bfloat16* base_ptr = static_cast<__nv_bfloat16*>(dst.p[owner]);
      uint4* out = reinterpret_cast<uint4*>(base_ptr + ((b * dst_token_capacity + local_s) * heads_all +
                                                        (int64_t)my_rank * heads_per_rank) * head_dim);
      out[p] = v[u];
    }
  }
}

// FP8 variant of the gather (the reference's per-token output quantization, _float8_comm.py:6-44 with
// eps = 1e-4 and the scale stored as bf16): per (token, head) s = max(amax, 1e-4) / 448, e4m3(clamp(x * (1/s))),
// the owner receives bytes and bf16 scales and multiplies by the ROUNDED scale when it unpacks.
__global__ void __launch_bounds__(128)
    gather_tokens_fp8_kernel(const __nv_bfloat16* __restrict__ o, const PeerPtrs dst, const PeerPtrs dst_scale,
                             const PeerRows rows_of, int world, int my_rank, int64_t batch, int64_t tokens_all,
                             int64_t dst_token_capacity, int heads_per_rank, int heads_all, int head_dim) {
  const int lph = head_dim / 8;  // lanes per head: 8, 16 or 32
  const int row_packets = heads_per_rank * lph;
  const int64_t rows = batch * tokens_all;
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const int64_t b = r / tokens_all, s = r - b * tokens_all;
    int owner = 0;
    while (owner + 1 < world && s >= rows_of.start[owner + 1]) ++owner;
    const int64_t local_s = s - rows_of.start[owner];
    const uint4* src = reinterpret_cast<const uint4*>(o + r * (int64_t)heads_per_rank * head_dim);
    const int64_t dst_head0 = (b * dst_token_capacity + local_s) * heads_all + (int64_t)my_rank * heads_per_rank;
    uint8_t* out8 = static_cast<uint8_t*>(dst.p[owner]) + dst_head0 * head_dim;
    __nv_bfloat16* out_s = static_cast<__nv_bfloat16*>(dst_scale.p[owner]) + dst_head0;
    const int passes = (row_packets + 127) / 128;
    for (int pass = 0; pass < passes; ++pass) {  // uniform trip count: the shuffles need whole warps
      const int p = pass * 128 + threadIdx.x;
      const uint4 v = p < row_packets ? __ldcs(src + p) : make_uint4(0, 0, 0, 0);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
      __nv_bfloat162 m2 = __habs2(pu2b(w[0]));
#pragma unroll
      for (int i = 1; i < 4; ++i) m2 = __hmax2(m2, __habs2(pu2b(w[i])));
      const uint32_t mu = pb2u(m2);
      float amax = fmaxf(__uint_as_float(mu << 16), __uint_as_float(mu & 0xffff0000u));
      for (int off = lph / 2; off > 0; off >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
      const float sc = __fdiv_rn(fmaxf(amax, 1e-4f), 448.0f);
      const float inv = __fdiv_rn(1.0f, sc);
      if (p < row_packets) {
        uint32_t q[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const uint32_t a = w[2 * h], b2 = w[2 * h + 1];
          const uint32_t lo = __nv_cvt_float2_to_fp8x2(
              make_float2(__fmul_rn(__uint_as_float(a << 16), inv), __fmul_rn(__uint_as_float(a & 0xffff0000u), inv)),
              __NV_SATFINITE, __NV_E4M3);
          const uint32_t hi = __nv_cvt_float2_to_fp8x2(
              make_float2(__fmul_rn(__uint_as_float(b2 << 16), inv), __fmul_rn(__uint_as_float(b2 & 0xffff0000u), inv)),
              __NV_SATFINITE, __NV_E4M3);
          q[h] = lo | (hi << 16);
        }
        *reinterpret_cast<uint2*>(out8 + (int64_t)p * 8) = make_uint2(q[0], q[1]);
        if (p % lph == 0) out_s[p / lph] = __float2bfloat16_rn(sc);
      }
    }
  }
}

// Unpack e4m3 rows of `head_dim` bytes with one scale each into bf16: out = bf16(float(q) * scale).
// SCALE_T = float (q / k / v) or __nv_bfloat16 (attention output).  Up to 3 tensors per launch.
struct DequantJobs {
  const uint8_t* q[3];
  const void* scale[3];
  __nv_bfloat16* out[3];
  int64_t rows[3];
};
template <typename SCALE_T>
__device__ __forceinline__ void dequant_packet(const uint4 v, float s, uint4* dst) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
  uint32_t o[8];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[k] & 0xffffu), __NV_E4M3);
    const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w[k] >> 16), __NV_E4M3);
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
    const float2 b2 = __half22float2(*reinterpret_cast<const __half2*>(&hi));
    o[2 * k] = pb2u(__floats2bfloat162_rn(__fmul_rn(a.x, s), __fmul_rn(a.y, s)));
    o[2 * k + 1] = pb2u(__floats2bfloat162_rn(__fmul_rn(b2.x, s), __fmul_rn(b2.y, s)));
  }
  __stcs(dst, make_uint4(o[0], o[1], o[2], o[3]));
  __stcs(dst + 1, make_uint4(o[4], o[5], o[6], o[7]));
}

// 16 bytes in, 32 bytes out per packet; four packets (a grid stride apart) in flight per thread.
constexpr int DQ_UNROLL = 4;
template <typename SCALE_T>
__global__ void __launch_bounds__(256)
    dequant_heads_kernel(const __grid_constant__ DequantJobs jobs, int head_dim) {
  const int j = blockIdx.y;
  const int pk_per_row = head_dim / 16;
  const int64_t total = jobs.rows[j] * pk_per_row;
  const uint4* src = reinterpret_cast<const uint4*>(jobs.q[j]);
  const SCALE_T* sc = static_cast<const SCALE_T*>(jobs.scale[j]);
  uint4* dst = reinterpret_cast<uint4*>(jobs.out[j]);
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += DQ_UNROLL * stride) {
    uint4 v[DQ_UNROLL];
    float s[DQ_UNROLL];
#pragma unroll
    for (int u = 0; u < DQ_UNROLL; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) {
        v[u] = __ldcs(src + i);
        s[u] = (float)sc[i / pk_per_row];
      }
    }
#pragma unroll
    for (int u = 0; u < DQ_UNROLL; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < total) dequant_packet<SCALE_T>(v[u], s[u], dst + 2 * i);
    }
  }
}

// ---- cross-GPU ordering ------------------------------------------------------------------------
// Flags: every rank owns `world` 32-bit words; word r of rank p's array is written by rank r only.
// Each rank keeps an epoch counter in its own memory.  signal: epoch += 1, then store the epoch into
// word `my_rank` of every rank's array (release at system scope; the data kernels before it on the
// stream have completed, so their stores to peer memory are already performed).  wait: spin until
// every word of the own array has reached the own epoch, bounded by a timeout; on expiry a sticky
// status is recorded and this and all later waits return at once, so a lost peer cannot hang the GPU.
struct PeerSync {
  unsigned int epoch;
  int status;  // 0 ok; 1 + peer index that was late
};

__global__ void peer_signal_kernel(const PeerPtrs flags, int my_rank, int world, PeerSync* sync) {
  __shared__ unsigned int e;
  if (threadIdx.x == 0) {
    e = sync->epoch + 1;
    sync->epoch = e;
  }
  __syncthreads();
  if ((int)threadIdx.x < world) {
    // st.release.sys = fence.acq_rel.sys + store: it alone orders everything that happened before this thread
    // (the earlier kernels' stores to peer memory included: they happen-before through the kernel boundary) in
    // front of the flag; a __threadfence_system() of its own here was a second 2 us fence per signal
    unsigned int* word = static_cast<unsigned int*>(flags.p[threadIdx.x]) + my_rank;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(word), "r"(e) : "memory");
  }
}

__global__ void peer_wait_kernel(const unsigned int* __restrict__ my_flags, int world, PeerSync* sync,
                                 unsigned long long timeout_ns) {
  if ((int)threadIdx.x >= world) return;
  if (sync->status != 0) return;  // sticky: a peer was lost earlier
  const unsigned int want = sync->epoch;
  const unsigned int* word = my_flags + threadIdx.x;
  unsigned long long t0 = 0;
  for (unsigned int it = 0;; ++it) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(word) : "memory");
    if ((int)(v - want) >= 0) break;  // epochs wrap: compare as a signed difference
    if ((it & 63u) == 63u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) {
        atomicCAS(&sync->status, 0, 1 + (int)threadIdx.x);
        break;
      }
      __nanosleep(200);
    }
  }
  // ld.acquire.sys = load + fence.acq_rel.sys: later reads of this thread, and through the kernel boundary of the
  // kernels that follow, are ordered behind the flag; no further fence is needed
}

// signal + wait in one launch (what a rank runs between the phases of the exchange).
__global__ void peer_barrier_kernel(const PeerPtrs flags, const unsigned int* __restrict__ my_flags, int my_rank,
                                    int world, PeerSync* sync, unsigned long long timeout_ns) {
  __shared__ unsigned int e;
  if (threadIdx.x == 0) {
    e = sync->epoch + 1;
    sync->epoch = e;
  }
  __syncthreads();
  if ((int)threadIdx.x >= world) return;
  unsigned int* word = static_cast<unsigned int*>(flags.p[threadIdx.x]) + my_rank;
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(word), "r"(e) : "memory");  // release = fence + store
  if (sync->status != 0) return;
  const unsigned int* mine = my_flags + threadIdx.x;
  unsigned long long t0 = 0;
  for (unsigned int it = 0;; ++it) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if ((int)(v - e) >= 0) break;
    if ((it & 63u) == 63u) {
      unsigned long long now;
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
      if (t0 == 0) t0 = now;
      else if (now - t0 > timeout_ns) {
        atomicCAS(&sync->status, 0, 1 + (int)threadIdx.x);
        break;
      }
      __nanosleep(200);
    }
  }
}

}  // namespace cdb

using namespace cdb;

static bool fill_ptrs(PeerPtrs* out, void* const* ptrs, int world) {
  if (!ptrs || world < 1 || world > PEER_MAX) return false;
  for (int i = 0; i < PEER_MAX; ++i) out->p[i] = i < world ? ptrs[i] : nullptr;
  for (int i = 0; i < world; ++i)
    if (!out->p[i] || !aligned16(out->p[i])) return false;
  return true;
}

extern "C" int cdb_peer_enable_access(int peer_device) {
  int dev = 0;
  CDB_CUDA_CHECK(cudaGetDevice(&dev));
  if (peer_device == dev) return CDB_OK;
  int can = 0;
  CDB_CUDA_CHECK(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return CDB_ERR_UNSUPPORTED;
  cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();
    return CDB_OK;
  }
  CDB_CUDA_CHECK(e);
  return CDB_OK;
}

// ---- buffers that peers can map ------------------------------------------------------------------
// Plain cudaMalloc allocations (one IPC handle = one buffer, offset 0), zero-filled.
extern "C" int cdb_peer_alloc(size_t bytes, void** out) {
  if (!out || bytes == 0) return CDB_ERR_BAD_ARGUMENT;
  void* p = nullptr;
  CDB_CUDA_CHECK(cudaMalloc(&p, bytes));
  cudaError_t e = cudaMemset(p, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    cudaFree(p);
    CDB_CUDA_CHECK(e);
  }
  *out = p;
  return CDB_OK;
}

extern "C" int cdb_peer_free(void* p) {
  if (p) CDB_CUDA_CHECK(cudaFree(p));
  return CDB_OK;
}

extern "C" int cdb_peer_export(const void* p, unsigned char* handle64) {
  if (!p || !handle64) return CDB_ERR_BAD_ARGUMENT;
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  CDB_CUDA_CHECK(cudaIpcGetMemHandle(&h, const_cast<void*>(p)));
  memcpy(handle64, &h, 64);
  return CDB_OK;
}

extern "C" int cdb_peer_import(const unsigned char* handle64, void** out) {
  if (!handle64 || !out) return CDB_ERR_BAD_ARGUMENT;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  CDB_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return CDB_OK;
}

extern "C" int cdb_peer_release(void* imported) {
  if (imported) CDB_CUDA_CHECK(cudaIpcCloseMemHandle(imported));
  return CDB_OK;
}

extern "C" int cdb_scatter_heads(const void* x, int64_t ld_x, const void* norm_weight, int norm_across_heads,
                                 const void* cos_table, const void* sin_table, int table_row_offset,
                                 void* const* dst_ptrs, int world,
                                 int64_t dst_batch_stride, int64_t tokens, int64_t tokens_per_batch,
                                 int64_t dst_row_offset, int heads, int head_dim, float eps, void* stream) {
  PeerPtrs dst;
  if (!x || tokens < 0 || tokens_per_batch <= 0 || heads <= 0 || !fill_ptrs(&dst, dst_ptrs, world))
    return CDB_ERR_BAD_ARGUMENT;
  const bool norm = norm_weight != nullptr;
  if (norm && (!cos_table || !sin_table)) return CDB_ERR_BAD_ARGUMENT;
  if (tokens == 0) return CDB_OK;
  if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || heads % world != 0 || ld_x % 8 != 0 ||
      dst_batch_stride % 8 != 0 || !aligned16(x) ||
      (norm && (!aligned16(norm_weight) || !aligned16(cos_table) || !aligned16(sin_table))))
    return CDB_ERR_UNSUPPORTED;
  const int hpr = heads / world;
  const int64_t ld_out = (int64_t)hpr * head_dim;
  const int64_t cap = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(tokens < cap ? tokens : cap);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(norm_weight);
  const __nv_bfloat16* cp = static_cast<const __nv_bfloat16*>(cos_table);
  const __nv_bfloat16* sp = static_cast<const __nv_bfloat16*>(sin_table);
#define CDB_SC(LPH, MODE)                                                                                     \
  scatter_heads_kernel<LPH, MODE><<<grid, SC_THREADS, 0, st>>>(xp, ld_x, wp, cp, sp, table_row_offset, dst, hpr, \
                                                               ld_out, dst_batch_stride, tokens, tokens_per_batch, \
                                                               dst_row_offset, heads, eps)
#define CDB_SC_DIM(MODE)                  \
  if (head_dim == 64) CDB_SC(8, MODE);    \
  else if (head_dim == 128) CDB_SC(16, MODE); \
  else CDB_SC(32, MODE)
  if (!norm) { CDB_SC_DIM(SCATTER_COPY); }
  else if (norm_across_heads) { CDB_SC_DIM(SCATTER_ROW_NORM); }
  else { CDB_SC_DIM(SCATTER_HEAD_NORM); }
#undef CDB_SC_DIM
#undef CDB_SC
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

struct cdb_scatter_job_abi {  // mirrors `cdb_scatter_job` of the public header
  const void* x;
  int64_t ld_x, tokens, tokens_per_batch;
  const void* norm_weight;
  int norm_across_heads;
  float eps;
  const void* cos_table;
  const void* sin_table;
  int table_row_offset;
  void* const* dst_ptrs;
  int64_t dst_batch_stride, dst_row_offset;
  void* const* dst_scale_ptrs;  // non-NULL: FP8 bytes go to dst_ptrs, one float32 scale per (token, head) here
};

extern "C" int cdb_scatter_heads_multi(const void* jobs_v, int njobs, int world, int heads, int head_dim, void* stream) {
  const cdb_scatter_job_abi* jobs = static_cast<const cdb_scatter_job_abi*>(jobs_v);
  if (!jobs || njobs < 1 || njobs > SCATTER_MAX_JOBS || heads <= 0 || world < 1 || world > PEER_MAX)
    return CDB_ERR_BAD_ARGUMENT;
  if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || heads % world != 0) return CDB_ERR_UNSUPPORTED;
  ScatterJobs packed{};
  int64_t max_tokens = 0;
  for (int i = 0; i < njobs; ++i) {
    const cdb_scatter_job_abi& in = jobs[i];
    ScatterJob& o = packed.job[i];
    if (!in.x || in.tokens < 0 || in.tokens_per_batch <= 0 || !fill_ptrs(&o.dst, in.dst_ptrs, world))
      return CDB_ERR_BAD_ARGUMENT;
    const bool norm = in.norm_weight != nullptr;
    if (norm && (!in.cos_table || !in.sin_table)) return CDB_ERR_BAD_ARGUMENT;
    if (in.ld_x % 8 != 0 || in.dst_batch_stride % 8 != 0 || !aligned16(in.x) ||
        (norm && (!aligned16(in.norm_weight) || !aligned16(in.cos_table) || !aligned16(in.sin_table))))
      return CDB_ERR_UNSUPPORTED;
    o.x = static_cast<const __nv_bfloat16*>(in.x);
    o.w = static_cast<const __nv_bfloat16*>(in.norm_weight);
    o.cs = static_cast<const __nv_bfloat16*>(in.cos_table);
    o.sn = static_cast<const __nv_bfloat16*>(in.sin_table);
    o.ld_x = in.ld_x;
    o.out_batch_stride = in.dst_batch_stride;
    o.tokens = in.tokens;
    o.tokens_per_batch = in.tokens_per_batch;
    o.dst_row_offset = in.dst_row_offset;
    o.table_row_offset = in.table_row_offset;
    o.mode = !norm ? SCATTER_COPY : (in.norm_across_heads ? SCATTER_ROW_NORM : SCATTER_HEAD_NORM);
    o.eps = in.eps;
    o.fp8_out = in.dst_scale_ptrs != nullptr;
    if (o.fp8_out && !fill_ptrs(&o.dst_scale, in.dst_scale_ptrs, world)) return CDB_ERR_BAD_ARGUMENT;
    max_tokens = in.tokens > max_tokens ? in.tokens : max_tokens;
  }
  if (max_tokens == 0) return CDB_OK;
  const int hpr = heads / world;
  const int64_t ld_out = (int64_t)hpr * head_dim;
  const int64_t cap = (int64_t)sm_count() * 16 / njobs + 1;
  const dim3 grid((unsigned)(max_tokens < cap ? max_tokens : cap), (unsigned)njobs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (head_dim == 64) scatter_heads_multi_kernel<8><<<grid, SC_THREADS, 0, st>>>(packed, hpr, ld_out, heads);
  else if (head_dim == 128) scatter_heads_multi_kernel<16><<<grid, SC_THREADS, 0, st>>>(packed, hpr, ld_out, heads);
  else scatter_heads_multi_kernel<32><<<grid, SC_THREADS, 0, st>>>(packed, hpr, ld_out, heads);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_peer_barrier(void* const* flag_ptrs, const void* my_flags, int world, int my_rank, void* sync,
                                uint64_t timeout_ns, void* stream) {
  PeerPtrs flags;
  if (!sync || !my_flags || my_rank < 0 || my_rank >= world || !fill_ptrs(&flags, flag_ptrs, world))
    return CDB_ERR_BAD_ARGUMENT;
  peer_barrier_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      flags, static_cast<const unsigned int*>(my_flags), my_rank, world, static_cast<PeerSync*>(sync),
      (unsigned long long)timeout_ns);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_gather_tokens(const void* o, void* const* dst_ptrs, int world, int my_rank, int64_t batch,
                                 int64_t tokens_all, const int64_t* row_starts, int64_t dst_token_capacity,
                                 int heads_per_rank, int head_dim, void* stream) {
  PeerPtrs dst;
  if (!o || batch <= 0 || tokens_all <= 0 || heads_per_rank <= 0 || my_rank < 0 || my_rank >= world ||
      !fill_ptrs(&dst, dst_ptrs, world))
    return CDB_ERR_BAD_ARGUMENT;
  if ((heads_per_rank * head_dim) % 8 != 0 || !aligned16(o)) return CDB_ERR_UNSUPPORTED;
  PeerRows rows_of{};
  if (row_starts) {
    for (int r = 0; r <= world; ++r) rows_of.start[r] = row_starts[r];
    if (rows_of.start[0] != 0 || rows_of.start[world] != tokens_all) return CDB_ERR_BAD_ARGUMENT;
    for (int r = 0; r < world; ++r) {
      const int64_t len = rows_of.start[r + 1] - rows_of.start[r];
      if (len < 0 || len > dst_token_capacity) return CDB_ERR_BAD_ARGUMENT;
    }
  } else {  // equal ranges
    if (tokens_all % world != 0) return CDB_ERR_BAD_ARGUMENT;
    for (int r = 0; r <= world; ++r) rows_of.start[r] = tokens_all / world * r;
    if (dst_token_capacity < tokens_all / world) return CDB_ERR_BAD_ARGUMENT;
  }
  const int64_t rows = batch * tokens_all;
  const int64_t cap = (int64_t)sm_count() * 16;
  const int64_t packets = rows * (heads_per_rank * head_dim / 8);
  const int64_t want = (packets + 256 * GT_UNROLL - 1) / (256 * GT_UNROLL);
  gather_tokens_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), dst, rows_of, world, my_rank, batch, tokens_all, dst_token_capacity,
      heads_per_rank, heads_per_rank * world, head_dim);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_gather_tokens_fp8(const void* o, void* const* dst_ptrs, void* const* dst_scale_ptrs, int world,
                                     int my_rank, int64_t batch, int64_t tokens_all, const int64_t* row_starts,
                                     int64_t dst_token_capacity, int heads_per_rank, int head_dim, void* stream) {
  PeerPtrs dst, dst_scale;
  if (!o || batch <= 0 || tokens_all <= 0 || heads_per_rank <= 0 || my_rank < 0 || my_rank >= world ||
      !fill_ptrs(&dst, dst_ptrs, world) || !fill_ptrs(&dst_scale, dst_scale_ptrs, world))
    return CDB_ERR_BAD_ARGUMENT;
  if ((head_dim != 64 && head_dim != 128 && head_dim != 256) || !aligned16(o)) return CDB_ERR_UNSUPPORTED;
  PeerRows rows_of{};
  if (row_starts) {
    for (int r = 0; r <= world; ++r) rows_of.start[r] = row_starts[r];
    if (rows_of.start[0] != 0 || rows_of.start[world] != tokens_all) return CDB_ERR_BAD_ARGUMENT;
  } else {
    if (tokens_all % world != 0) return CDB_ERR_BAD_ARGUMENT;
    for (int r = 0; r <= world; ++r) rows_of.start[r] = tokens_all / world * r;
  }
  for (int r = 0; r < world; ++r)
    if (rows_of.start[r + 1] - rows_of.start[r] < 0 || rows_of.start[r + 1] - rows_of.start[r] > dst_token_capacity)
      return CDB_ERR_BAD_ARGUMENT;
  const int64_t rows = batch * tokens_all;
  const int64_t cap = (int64_t)sm_count() * 16;
  gather_tokens_fp8_kernel<<<(unsigned)(rows < cap ? rows : cap), 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), dst, dst_scale, rows_of, world, my_rank, batch, tokens_all,
      dst_token_capacity, heads_per_rank, heads_per_rank * world, head_dim);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_fp8_dequant_heads(const void* const* q, const void* const* scales, void* const* out,
                                     const int64_t* rows, int njobs, int head_dim, int scales_are_bf16, void* stream) {
  if (!q || !scales || !out || !rows || njobs < 1 || njobs > 3) return CDB_ERR_BAD_ARGUMENT;
  if (head_dim % 16 != 0) return CDB_ERR_UNSUPPORTED;
  DequantJobs jobs{};
  int64_t max_rows = 0;
  for (int i = 0; i < njobs; ++i) {
    if (!q[i] || !scales[i] || !out[i] || rows[i] < 0) return CDB_ERR_BAD_ARGUMENT;
    if (!aligned16(q[i]) || !aligned16(out[i])) return CDB_ERR_UNSUPPORTED;
    jobs.q[i] = static_cast<const uint8_t*>(q[i]);
    jobs.scale[i] = scales[i];
    jobs.out[i] = static_cast<__nv_bfloat16*>(out[i]);
    jobs.rows[i] = rows[i];
    max_rows = rows[i] > max_rows ? rows[i] : max_rows;
  }
  if (max_rows == 0) return CDB_OK;
  const int64_t total = max_rows * (head_dim / 16);
  const int64_t want = (total + 256 * DQ_UNROLL - 1) / (256 * DQ_UNROLL);
  const int64_t cap = (int64_t)sm_count() * 8;
  const dim3 grid((unsigned)(want < cap ? want : cap), (unsigned)njobs);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (scales_are_bf16) dequant_heads_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(jobs, head_dim);
  else dequant_heads_kernel<float><<<grid, 256, 0, st>>>(jobs, head_dim);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" size_t cdb_peer_sync_bytes(void) { return sizeof(PeerSync); }

extern "C" int cdb_peer_signal(void* const* flag_ptrs, int world, int my_rank, void* sync, void* stream) {
  PeerPtrs flags;
  if (!sync || my_rank < 0 || my_rank >= world || !fill_ptrs(&flags, flag_ptrs, world)) return CDB_ERR_BAD_ARGUMENT;
  peer_signal_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(flags, my_rank, world,
                                                                      static_cast<PeerSync*>(sync));
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_peer_wait(const void* my_flags, int world, void* sync, uint64_t timeout_ns, void* stream) {
  if (!my_flags || !sync || world < 1 || world > PEER_MAX) return CDB_ERR_BAD_ARGUMENT;
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const unsigned int*>(my_flags), world,
                                                                    static_cast<PeerSync*>(sync),
                                                                    (unsigned long long)timeout_ns);
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}
