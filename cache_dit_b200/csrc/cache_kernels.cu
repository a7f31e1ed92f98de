// DBCache / TaylorSeer step kernels for sm_100a: single-pass, 128-bit vectorised streaming.
//
//   rel_l1_kernel        Fn-residual formation + the two means of the relative-L1 check
//   taylor_apply_kernel  Taylor extrapolation of the cached residual + add to hidden states
//   taylor_update_kernel Mn-residual formation + finite-difference derivative ladder
//
// All three are HBM-bound (no reuse), so the design goals are: touch every byte once, keep
// >= 4 independent 16-byte loads in flight per thread, size the grid to one resident wave.
// Arithmetic mirrors the reference's eager PyTorch op-by-op rounding (each elementwise op
// materialises a tensor in the storage dtype), which is what keeps hit/miss decisions
// bit-identical in bf16.
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace cdb {

// ------------------------------------------------------------------------------------------
// relative-L1 reduction
// ------------------------------------------------------------------------------------------
constexpr int RL_THREADS = 512;
constexpr int RL_CLUSTER = 2;        // CTA pair: always fits (SMs come in TPC pairs)
constexpr int RL_MAX_CLUSTERS = 1024;
constexpr int RL_UNROLL = 2;

struct RelL1Scratch {
  unsigned int ticket;  // clusters finished in the current launch; self-resetting
  unsigned int pad[3];
  double partial[RL_MAX_CLUSTERS][2];
};

template <typename T, int W>
struct Chunk {  // W elements: W == VEC -> one 16-byte access, W == 1 -> scalar fallback
  T v[W];
};

template <typename T, int W>
__device__ __forceinline__ Chunk<T, W> load_chunk(const T* p) {
  Chunk<T, W> c;
  if constexpr (W == 1) {
    c.v[0] = *p;
  } else {
    Pack<T> k = ld_stream(p);
#pragma unroll
    for (int i = 0; i < W; ++i) c.v[i] = k.v[i];
  }
  return c;
}
template <typename T, int W>
__device__ __forceinline__ void store_chunk(T* p, const Chunk<T, W>& c) {
  if constexpr (W == 1) {
    *p = c.v[0];
  } else {
    Pack<T> k;
#pragma unroll
    for (int i = 0; i < W; ++i) k.v[i] = c.v[i];
    st_stream(p, k);
  }
}

template <typename T, int W, bool HAS_BASE, bool HAS_PREV, bool WRITE_RES>
__device__ __forceinline__ void rel_l1_chunk(const T* cur, const T* base, const T* prev, T* res,
                                             int64_t off, float& sd, float& sp) {
  Chunk<T, W> c = load_chunk<T, W>(cur + off);
  Chunk<T, W> b, p, r;
  if constexpr (HAS_BASE) b = load_chunk<T, W>(base + off);
  if constexpr (HAS_PREV) p = load_chunk<T, W>(prev + off);
#pragma unroll
  for (int i = 0; i < W; ++i) {
    float rv = DT<T>::load(c.v[i]);
    if constexpr (HAS_BASE) rv = DT<T>::round(__fsub_rn(rv, DT<T>::load(b.v[i])));
    if constexpr (WRITE_RES) r.v[i] = DT<T>::store(rv);
    if constexpr (HAS_PREV) {
      float pv = DT<T>::load(p.v[i]);
      sd += fabsf(DT<T>::round(__fsub_rn(pv, rv)));
      sp += fabsf(pv);
    }
  }
  if constexpr (WRITE_RES) store_chunk<T, W>(res + off, r);
}

template <typename T, int W, bool HAS_BASE, bool HAS_PREV, bool WRITE_RES>
__global__ void __cluster_dims__(RL_CLUSTER, 1, 1) __launch_bounds__(RL_THREADS)
    rel_l1_kernel(const T* __restrict__ cur, const T* __restrict__ base,
                  const T* __restrict__ prev, T* __restrict__ res, int64_t n,
                  float* __restrict__ means, RelL1Scratch* __restrict__ scratch) {
  const int64_t nchunk = n / W;
  const int64_t stride = (int64_t)gridDim.x * RL_THREADS;
  // Four accumulators: two per unrolled lane, so the adds do not serialise behind the loads.
  float sd[RL_UNROLL] = {0.f, 0.f}, sp[RL_UNROLL] = {0.f, 0.f};
  int64_t i = (int64_t)blockIdx.x * RL_THREADS + threadIdx.x;
  for (; i + stride < nchunk; i += RL_UNROLL * stride) {
#pragma unroll
    for (int u = 0; u < RL_UNROLL; ++u)
      rel_l1_chunk<T, W, HAS_BASE, HAS_PREV, WRITE_RES>(cur, base, prev, res, (i + u * stride) * W,
                                                        sd[u], sp[u]);
  }
  if (i < nchunk)
    rel_l1_chunk<T, W, HAS_BASE, HAS_PREV, WRITE_RES>(cur, base, prev, res, i * W, sd[0], sp[0]);
  if constexpr (W > 1) {  // ragged tail (< W elements), one thread
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int64_t t = nchunk * W; t < n; ++t)
        rel_l1_chunk<T, 1, HAS_BASE, HAS_PREV, WRITE_RES>(cur, base, prev, res, t, sd[1], sp[1]);
  }
  if constexpr (!HAS_PREV) return;

  // thread -> warp (shuffle) -> CTA (shared memory) -> cluster (distributed shared memory)
  float d = warp_sum(sd[0] + sd[1]);
  float p = warp_sum(sp[0] + sp[1]);
  __shared__ float s_warp[RL_THREADS / 32][2];
  __shared__ double s_cta[RL_CLUSTER][2];  // slot r is written by cluster rank r (only rank 0's is read)
  __shared__ int s_last;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_warp[warp][0] = d;
    s_warp[warp][1] = p;
  }
  __syncthreads();
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned rank = cluster.block_rank();
  if (warp == 0) {
    float bd = lane < RL_THREADS / 32 ? s_warp[lane][0] : 0.f;
    float bp = lane < RL_THREADS / 32 ? s_warp[lane][1] : 0.f;
    bd = warp_sum(bd);
    bp = warp_sum(bp);
    if (lane == 0) {
      double* dst = cluster.map_shared_rank(&s_cta[0][0], 0);  // rank 0's copy of s_cta
      dst[rank * 2 + 0] = (double)bd;
      dst[rank * 2 + 1] = (double)bp;
    }
  }
  cluster.sync();  // hardware cluster barrier: every CTA of the pair arrives exactly once
  if (rank != 0) return;

  const unsigned nclusters = gridDim.x / RL_CLUSTER;
  const unsigned cid = blockIdx.x / RL_CLUSTER;
  if (threadIdx.x == 0) {
    double td = 0.0, tp = 0.0;
#pragma unroll
    for (int r = 0; r < RL_CLUSTER; ++r) {
      td += s_cta[r][0];
      tp += s_cta[r][1];
    }
    scratch->partial[cid][0] = td;
    scratch->partial[cid][1] = tp;
    __threadfence();
    unsigned t = atomicAdd(&scratch->ticket, 1u);
    s_last = (t == nclusters - 1);
  }
  __syncthreads();
  if (!s_last || warp != 0) return;
  // Last cluster to finish folds the partials in a fixed order (run-to-run deterministic).
  __threadfence();
  double td = 0.0, tp = 0.0;
  for (unsigned c = lane; c < nclusters; c += 32) {
    td += __ldcg(&scratch->partial[c][0]);
    tp += __ldcg(&scratch->partial[c][1]);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    td += __shfl_xor_sync(0xffffffffu, td, o);
    tp += __shfl_xor_sync(0xffffffffu, tp, o);
  }
  if (lane == 0) {
    means[0] = DT<T>::round((float)(td / (double)n));
    means[1] = DT<T>::round((float)(tp / (double)n));
    scratch->ticket = 0;  // ready for the next launch on this stream
  }
}

template <typename T, int W>
static int launch_rel_l1(const void* cur, const void* base, const void* prev, void* res, int64_t n,
                         float* means, RelL1Scratch* scratch, cudaStream_t st) {
  const int64_t nchunk = n / W;
  int64_t want = (nchunk + (int64_t)RL_THREADS * RL_UNROLL - 1) / ((int64_t)RL_THREADS * RL_UNROLL);
  int64_t cap = (int64_t)sm_count() * (2048 / RL_THREADS);  // one resident wave
  if (cap > RL_MAX_CLUSTERS * RL_CLUSTER) cap = RL_MAX_CLUSTERS * RL_CLUSTER;
  int64_t grid = want < cap ? want : cap;
  grid = (grid + RL_CLUSTER - 1) / RL_CLUSTER * RL_CLUSTER;
  if (grid < RL_CLUSTER) grid = RL_CLUSTER;
  const T* c = static_cast<const T*>(cur);
  const T* b = static_cast<const T*>(base);
  const T* p = static_cast<const T*>(prev);
  T* r = static_cast<T*>(res);
#define CDB_RL(HB, HP, WR) \
  rel_l1_kernel<T, W, HB, HP, WR><<<(unsigned)grid, RL_THREADS, 0, st>>>(c, b, p, r, n, means, scratch)
  const bool hb = base != nullptr, hp = prev != nullptr, wr = res != nullptr;
  if (hb && hp && wr) CDB_RL(true, true, true);
  else if (hb && hp && !wr) CDB_RL(true, true, false);
  else if (hb && !hp && wr) CDB_RL(true, false, true);
  else if (!hb && hp && wr) CDB_RL(false, true, true);
  else if (!hb && hp && !wr) CDB_RL(false, true, false);
  else if (!hb && !hp && wr) CDB_RL(false, false, true);
  else return CDB_ERR_BAD_ARGUMENT;  // nothing to compute
#undef CDB_RL
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

// ------------------------------------------------------------------------------------------
// elementwise kernels: Taylor apply and Taylor update
// ------------------------------------------------------------------------------------------
constexpr int EW_THREADS = 256;
constexpr int EW_UNROLL = 2;

struct ApplyArgs {
  const void* deriv[CDB_MAX_TAYLOR_TERMS];
  float coef[CDB_MAX_TAYLOR_TERMS];
  float power[CDB_MAX_TAYLOR_TERMS];
};

template <typename T, int W, int TERMS, bool ADD>
__device__ __forceinline__ void apply_chunk(const T* hidden, const ApplyArgs& a, T* out, int64_t off) {
  Chunk<T, W> h, o, d[TERMS];
  if constexpr (ADD) h = load_chunk<T, W>(hidden + off);
#pragma unroll
  for (int t = 0; t < TERMS; ++t) d[t] = load_chunk<T, W>(static_cast<const T*>(a.deriv[t]) + off);
#pragma unroll
  for (int i = 0; i < W; ++i) {
    // output = 0; output += (1/t!) * dY[t] * elapsed**t  -- three rounded ops per term
    float acc = 0.f;
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
      float term = DT<T>::round(__fmul_rn(a.coef[t], DT<T>::load(d[t].v[i])));
      term = DT<T>::round(__fmul_rn(term, a.power[t]));
      acc = DT<T>::round(__fadd_rn(acc, term));
    }
    if constexpr (ADD) acc = DT<T>::round(__fadd_rn(acc, DT<T>::load(h.v[i])));
    o.v[i] = DT<T>::store(acc);
  }
  store_chunk<T, W>(out + off, o);
}

template <typename T, int W, int TERMS, bool ADD>
__global__ void __launch_bounds__(EW_THREADS)
    taylor_apply_kernel(const T* __restrict__ hidden, const __grid_constant__ ApplyArgs a,
                        T* __restrict__ out, int64_t n) {
  const int64_t nchunk = n / W;
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
  for (; i + stride < nchunk; i += EW_UNROLL * stride) {
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u)
      apply_chunk<T, W, TERMS, ADD>(hidden, a, out, (i + u * stride) * W);
  }
  if (i < nchunk) apply_chunk<T, W, TERMS, ADD>(hidden, a, out, i * W);
  if constexpr (W > 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int64_t t = nchunk * W; t < n; ++t) apply_chunk<T, 1, TERMS, ADD>(hidden, a, out, t);
  }
}

struct UpdateArgs {
  const void* prev[CDB_MAX_TAYLOR_TERMS];
  void* cur[CDB_MAX_TAYLOR_TERMS];
};

template <typename T, int W, int NEW, bool HAS_BEFORE, bool WRITE_Y>
__device__ __forceinline__ void update_chunk(const T* after, const T* before, const UpdateArgs& a,
                                             float window, int64_t off) {
  Chunk<T, W> y = load_chunk<T, W>(after + off);
  Chunk<T, W> b, p[NEW > 0 ? NEW : 1], o[NEW > 0 ? NEW : 1];
  if constexpr (HAS_BEFORE) b = load_chunk<T, W>(before + off);
#pragma unroll
  for (int k = 0; k < NEW; ++k) p[k] = load_chunk<T, W>(static_cast<const T*>(a.prev[k]) + off);
#pragma unroll
  for (int i = 0; i < W; ++i) {
    float v = DT<T>::load(y.v[i]);
    if constexpr (HAS_BEFORE) {
      v = DT<T>::round(__fsub_rn(v, DT<T>::load(b.v[i])));
      y.v[i] = DT<T>::store(v);
    }
#pragma unroll
    for (int k = 0; k < NEW; ++k) {
      // dY[k+1] = (dY[k] - dY_prev[k]) / window : a rounded subtraction, then a rounded division
      v = DT<T>::round(__fsub_rn(v, DT<T>::load(p[k].v[i])));
      v = DT<T>::round(__fdiv_rn(v, window));
      o[k].v[i] = DT<T>::store(v);
    }
  }
  if constexpr (WRITE_Y) store_chunk<T, W>(static_cast<T*>(a.cur[0]) + off, y);
#pragma unroll
  for (int k = 0; k < NEW; ++k) store_chunk<T, W>(static_cast<T*>(a.cur[k + 1]) + off, o[k]);
}

template <typename T, int W, int NEW, bool HAS_BEFORE, bool WRITE_Y>
__global__ void __launch_bounds__(EW_THREADS)
    taylor_update_kernel(const T* __restrict__ after, const T* __restrict__ before,
                         const __grid_constant__ UpdateArgs a, float window, int64_t n) {
  const int64_t nchunk = n / W;
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
  for (; i + stride < nchunk; i += EW_UNROLL * stride) {
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u)
      update_chunk<T, W, NEW, HAS_BEFORE, WRITE_Y>(after, before, a, window, (i + u * stride) * W);
  }
  if (i < nchunk) update_chunk<T, W, NEW, HAS_BEFORE, WRITE_Y>(after, before, a, window, i * W);
  if constexpr (W > 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int64_t t = nchunk * W; t < n; ++t)
        update_chunk<T, 1, NEW, HAS_BEFORE, WRITE_Y>(after, before, a, window, t);
  }
}

static unsigned ew_grid(int64_t nchunk) {
  int64_t want = (nchunk + (int64_t)EW_THREADS * EW_UNROLL - 1) / ((int64_t)EW_THREADS * EW_UNROLL);
  int64_t cap = (int64_t)sm_count() * (2048 / EW_THREADS);
  int64_t g = want < cap ? want : cap;
  return (unsigned)(g < 1 ? 1 : g);
}

template <typename T, int W>
static int launch_apply(const void* hidden, const ApplyArgs& a, int n_terms, bool add, void* out,
                        int64_t n, cudaStream_t st) {
  const unsigned grid = ew_grid(n / W);
  const T* h = static_cast<const T*>(hidden);
  T* o = static_cast<T*>(out);
#define CDB_AP(TERMS)                                                                        \
  case TERMS:                                                                                \
    if (add) taylor_apply_kernel<T, W, TERMS, true><<<grid, EW_THREADS, 0, st>>>(h, a, o, n); \
    else taylor_apply_kernel<T, W, TERMS, false><<<grid, EW_THREADS, 0, st>>>(h, a, o, n);    \
    break;
  switch (n_terms) {
    CDB_AP(1) CDB_AP(2) CDB_AP(3) CDB_AP(4) CDB_AP(5)
    default: return CDB_ERR_BAD_ARGUMENT;
  }
#undef CDB_AP
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

template <typename T, int W>
static int launch_update(const void* after, const void* before, const UpdateArgs& a, int n_new,
                         bool write_y, float window, int64_t n, cudaStream_t st) {
  const unsigned grid = ew_grid(n / W);
  const T* af = static_cast<const T*>(after);
  const T* bf = static_cast<const T*>(before);
  const bool hb = before != nullptr;
#define CDB_UP(NEW)                                                                                  \
  case NEW:                                                                                          \
    if (hb) taylor_update_kernel<T, W, NEW, true, true><<<grid, EW_THREADS, 0, st>>>(af, bf, a, window, n); \
    else if (write_y) taylor_update_kernel<T, W, NEW, false, true><<<grid, EW_THREADS, 0, st>>>(af, bf, a, window, n); \
    else taylor_update_kernel<T, W, NEW, false, false><<<grid, EW_THREADS, 0, st>>>(af, bf, a, window, n); \
    break;
  switch (n_new) {
    CDB_UP(0) CDB_UP(1) CDB_UP(2) CDB_UP(3) CDB_UP(4)
    default: return CDB_ERR_BAD_ARGUMENT;
  }
#undef CDB_UP
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

}  // namespace cdb

// ------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------
using namespace cdb;

extern "C" size_t cdb_rel_l1_scratch_bytes(void) { return sizeof(RelL1Scratch); }

extern "C" int cdb_rel_l1(const void* cur, const void* base, const void* prev, void* residual_out,
                          int64_t n, int dtype, float* means, void* scratch, size_t scratch_bytes,
                          void* stream) {
  if (!cur || n <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (!prev && !residual_out) return CDB_ERR_BAD_ARGUMENT;
  if (prev && (!means || !scratch)) return CDB_ERR_BAD_ARGUMENT;
  if (prev && scratch_bytes < sizeof(RelL1Scratch)) return CDB_ERR_SCRATCH_TOO_SMALL;
  if (residual_out && !base && residual_out == cur) residual_out = nullptr;  // nothing to copy
  if (!prev && !residual_out) return CDB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RelL1Scratch* sc = static_cast<RelL1Scratch*>(scratch);
  const bool vec = aligned16(cur) && aligned16(base) && aligned16(prev) && aligned16(residual_out);
  switch (dtype) {
    case CDB_F32:
      return vec ? launch_rel_l1<float, 4>(cur, base, prev, residual_out, n, means, sc, st)
                 : launch_rel_l1<float, 1>(cur, base, prev, residual_out, n, means, sc, st);
    case CDB_BF16:
      return vec ? launch_rel_l1<__nv_bfloat16, 8>(cur, base, prev, residual_out, n, means, sc, st)
                 : launch_rel_l1<__nv_bfloat16, 1>(cur, base, prev, residual_out, n, means, sc, st);
    case CDB_F16:
      return vec ? launch_rel_l1<__half, 8>(cur, base, prev, residual_out, n, means, sc, st)
                 : launch_rel_l1<__half, 1>(cur, base, prev, residual_out, n, means, sc, st);
    default:
      return CDB_ERR_BAD_ARGUMENT;
  }
}

extern "C" int cdb_taylor_apply(const void* hidden, const void* const* derivs, const float* coef,
                                const float* power, int n_terms, int add_hidden, void* out,
                                int64_t n, int dtype, void* stream) {
  if (!derivs || !coef || !power || !out || n <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (n_terms < 1 || n_terms > CDB_MAX_TAYLOR_TERMS) return CDB_ERR_BAD_ARGUMENT;
  if (add_hidden && !hidden) return CDB_ERR_BAD_ARGUMENT;
  ApplyArgs a{};
  bool vec = aligned16(out) && (!add_hidden || aligned16(hidden));
  for (int t = 0; t < n_terms; ++t) {
    if (!derivs[t]) return CDB_ERR_BAD_ARGUMENT;
    a.deriv[t] = derivs[t];
    a.coef[t] = coef[t];
    a.power[t] = power[t];
    vec = vec && aligned16(derivs[t]);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool add = add_hidden != 0;
  switch (dtype) {
    case CDB_F32:
      return vec ? launch_apply<float, 4>(hidden, a, n_terms, add, out, n, st)
                 : launch_apply<float, 1>(hidden, a, n_terms, add, out, n, st);
    case CDB_BF16:
      return vec ? launch_apply<__nv_bfloat16, 8>(hidden, a, n_terms, add, out, n, st)
                 : launch_apply<__nv_bfloat16, 1>(hidden, a, n_terms, add, out, n, st);
    case CDB_F16:
      return vec ? launch_apply<__half, 8>(hidden, a, n_terms, add, out, n, st)
                 : launch_apply<__half, 1>(hidden, a, n_terms, add, out, n, st);
    default:
      return CDB_ERR_BAD_ARGUMENT;
  }
}

extern "C" int cdb_taylor_update(const void* after, const void* before, const void* const* prev,
                                 void* const* cur, int n_new, float window, int64_t n, int dtype,
                                 void* stream) {
  if (!after || !cur || !cur[0] || n <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (n_new < 0 || n_new > CDB_MAX_TAYLOR_TERMS - 1) return CDB_ERR_BAD_ARGUMENT;
  if (n_new > 0 && (!prev || window == 0.f)) return CDB_ERR_BAD_ARGUMENT;
  UpdateArgs a{};
  bool vec = aligned16(after) && aligned16(before) && aligned16(cur[0]);
  a.cur[0] = cur[0];
  for (int k = 0; k < n_new; ++k) {
    if (!prev[k] || !cur[k + 1]) return CDB_ERR_BAD_ARGUMENT;
    for (int j = 0; j <= n_new; ++j)
      if (prev[k] == cur[j]) return CDB_ERR_BAD_ARGUMENT;  // ladder must be double-buffered
    a.prev[k] = prev[k];
    a.cur[k + 1] = cur[k + 1];
    vec = vec && aligned16(prev[k]) && aligned16(cur[k + 1]);
  }
  const bool write_y = before != nullptr || cur[0] != after;
  if (!write_y && n_new == 0) return CDB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  switch (dtype) {
    case CDB_F32:
      return vec ? launch_update<float, 4>(after, before, a, n_new, write_y, window, n, st)
                 : launch_update<float, 1>(after, before, a, n_new, write_y, window, n, st);
    case CDB_BF16:
      return vec ? launch_update<__nv_bfloat16, 8>(after, before, a, n_new, write_y, window, n, st)
                 : launch_update<__nv_bfloat16, 1>(after, before, a, n_new, write_y, window, n, st);
    case CDB_F16:
      return vec ? launch_update<__half, 8>(after, before, a, n_new, write_y, window, n, st)
                 : launch_update<__half, 1>(after, before, a, n_new, write_y, window, n, st);
    default:
      return CDB_ERR_BAD_ARGUMENT;
  }
}
