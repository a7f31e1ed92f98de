// DBCache / TaylorSeer step kernels for sm_100a: single-pass, 128-bit vectorised streaming.
//
//   rel_l1_kernel        Fn-residual formation + the two means of the relative-L1 check
//   taylor_apply_kernel  Taylor extrapolation of the cached residual + add to hidden states
//   taylor_update_kernel Mn-residual formation + finite-difference derivative ladder
//
// All three are HBM-bound (no reuse), so the design goals are: touch every byte once, keep
// >= 4 independent 16-byte loads in flight per thread, size the grid to one resident wave, and
// keep the instruction count per element low enough that issue never limits the stream.
// Arithmetic mirrors the reference's eager PyTorch op-by-op rounding (each elementwise op
// materialises a tensor in the storage dtype), which is what keeps hit/miss decisions
// bit-identical in bf16; the arithmetic policies in common.cuh do that with packed 16-bit
// hardware ops.
#include <cooperative_groups.h>

#include <cstdlib>
#include <mutex>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace cdb {

// CTAs of `kernel` that are resident at once on the whole device (one wave), from the occupancy
// calculator, so that a grid-stride launch never leaves a partial second wave behind.
template <class K>
static int64_t resident_ctas(K kernel, int threads) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, 0) != cudaSuccess || per_sm < 1)
    per_sm = 1;
  return (int64_t)per_sm * sm_count();
}

// CTAs of a cluster kernel that are guaranteed to be resident together (whole clusters).
template <class K>
static int64_t resident_cluster_ctas(K kernel, int threads, int cluster) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = dim3((unsigned)(cluster * 4096));
  cfg.blockDim = dim3((unsigned)threads);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = (unsigned)cluster;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  if (cudaOccupancyMaxActiveClusters(&clusters, kernel, &cfg) == cudaSuccess && clusters >= 1)
    return (int64_t)clusters * cluster;
  (void)cudaGetLastError();
  // fall back to half of the per-SM figure, rounded to whole clusters: conservative on purpose
  const int64_t ctas = resident_ctas(kernel, threads) / 2;
  return ctas / cluster * cluster >= cluster ? ctas / cluster * cluster : cluster;
}

// ------------------------------------------------------------------------------------------
// relative-L1 reduction
// ------------------------------------------------------------------------------------------
constexpr int RL_THREADS = 256;
constexpr int RL_CLUSTER = 2;        // default cluster: a CTA pair always fits (SMs come in TPC pairs)
constexpr int RL_CLUSTER_MAX = 8;    // largest cluster the kernel's shared buffers allow (CDB_RL_CLUSTER = 1, 2, 4, 8)
constexpr int RL_MAX_CLUSTERS = 1024;
constexpr int RL_UNROLL = 2;

// Reduction scratch: one record per cluster = the pair's two sums as fp64 bit patterns.  A word of all-zero
// bits means "not written yet" (a sum that is exactly zero is stored as -0.0, which has a non-zero pattern),
// so the data is its own ready flag: writers need no fence, no atomic and no ticket, and the folding CTA
// puts the zeros back when it has read a word, which is the state the next launch expects.
constexpr int RL_FOLD_WORDS = 2 * RL_MAX_CLUSTERS / RL_THREADS;  // words per thread of the folding CTA
struct RelL1Scratch {
  unsigned long long partial[RL_MAX_CLUSTERS][2];
};
constexpr unsigned long long RL_FOLD_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
template <class A, int U, bool HAS_BASE, bool HAS_PREV, bool WRITE_RES>
__device__ __forceinline__ void rel_l1_chunk(const typename A::T* cur, const typename A::T* base,
                                             const typename A::T* prev, typename A::T* res,
                                             int64_t off, float& sd, float& sp) {
  Chunk<A, U> r = load_chunk<A, U>(cur + off);
  Chunk<A, U> b, p;
  if constexpr (HAS_BASE) b = load_chunk<A, U>(base + off);
  if constexpr (HAS_PREV) p = load_chunk<A, U>(prev + off);
#pragma unroll
  for (int i = 0; i < U; ++i) {
    if constexpr (HAS_BASE) r.u[i] = A::sub(r.u[i], b.u[i]);  // Fn residual, rounded
    if constexpr (HAS_PREV) {
      A::accum(sd, A::abs(A::sub(p.u[i], r.u[i])));           // |round(prev - r)|
      A::accum(sp, A::abs(p.u[i]));                           // |prev|
    }
  }
  if constexpr (WRITE_RES) store_chunk<A, U>(res + off, r);
}

// A = vector policy with U units per 16 bytes, A1 = its one-element twin for the ragged tail.
template <class A, class A1, int U, bool HAS_BASE, bool HAS_PREV, bool WRITE_RES>
__global__ void __launch_bounds__(RL_THREADS)
    rel_l1_kernel(const typename A::T* __restrict__ cur, const typename A::T* __restrict__ base,
                  const typename A::T* __restrict__ prev, typename A::T* __restrict__ res, int64_t n,
                  float* __restrict__ means, RelL1Scratch* __restrict__ scratch) {
  constexpr int W = U * A::N;  // elements per chunk
  pdl_launch_dependents();
  pdl_wait_prior();
  const int64_t nchunk = n / W;
  const int64_t stride = (int64_t)gridDim.x * RL_THREADS;
  // Two accumulators per sum, one per unrolled lane, so the adds do not serialise.
  float sd[RL_UNROLL] = {0.f, 0.f}, sp[RL_UNROLL] = {0.f, 0.f};
  int64_t i = (int64_t)blockIdx.x * RL_THREADS + threadIdx.x;
  for (; i + stride < nchunk; i += RL_UNROLL * stride) {
#pragma unroll
    for (int u = 0; u < RL_UNROLL; ++u)
      rel_l1_chunk<A, U, HAS_BASE, HAS_PREV, WRITE_RES>(cur, base, prev, res, (i + u * stride) * W,
                                                        sd[u], sp[u]);
  }
  if (i < nchunk)
    rel_l1_chunk<A, U, HAS_BASE, HAS_PREV, WRITE_RES>(cur, base, prev, res, i * W, sd[0], sp[0]);
  if constexpr (W > 1) {  // ragged tail (< W elements), one thread
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int64_t t = nchunk * W; t < n; ++t)
        rel_l1_chunk<A1, 1, HAS_BASE, HAS_PREV, WRITE_RES>(cur, base, prev, res, t, sd[1], sp[1]);
  }
  if constexpr (!HAS_PREV) return;

  // thread -> warp (shuffle) -> CTA (shared memory) -> cluster (distributed shared memory)
  float d = warp_sum(sd[0] + sd[1]);
  float p = warp_sum(sp[0] + sp[1]);
  __shared__ float s_warp[RL_THREADS / 32][2];  // RL_THREADS / 32 <= 32 warps
  __shared__ double s_cta[RL_CLUSTER_MAX][2];  // only rank 0's copy is read; slot r is written by rank r
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    s_warp[warp][0] = d;
    s_warp[warp][1] = p;
  }
  __syncthreads();
  // The cluster size is a launch attribute (1 = no clusters): the kernel adapts to what it was launched with.
  cg::cluster_group cluster = cg::this_cluster();
  const unsigned csize = cluster.num_blocks();
  const unsigned rank = cluster.block_rank();
  if (warp == 0) {
    float bd = lane < RL_THREADS / 32 ? s_warp[lane][0] : 0.f;
    float bp = lane < RL_THREADS / 32 ? s_warp[lane][1] : 0.f;
    bd = warp_sum(bd);
    bp = warp_sum(bp);
    if (lane == 0) {
      double* dst = csize > 1 ? cluster.map_shared_rank(&s_cta[0][0], 0) : &s_cta[0][0];  // rank 0's copy of s_cta
      dst[rank * 2 + 0] = (double)bd;
      dst[rank * 2 + 1] = (double)bp;
    }
  }
  if (csize > 1) cluster.sync();  // hardware cluster barrier: every CTA of the cluster arrives exactly once
  if (rank != 0) return;

  // The pair's leader publishes its two fp64 sums with two plain 8-byte stores (single-copy atomic; the value
  // is its own ready flag, see RelL1Scratch).  Nothing is waited for: every cluster but the first is done here.
  const unsigned cid = blockIdx.x / csize;
  if (threadIdx.x == 0) {
    double td = 0.0, tp = 0.0;
    for (unsigned r = 0; r < csize; ++r) {
      td += s_cta[r][0];
      tp += s_cta[r][1];
    }
    st_relaxed_u64(&scratch->partial[cid][0], (unsigned long long)__double_as_longlong(td == 0.0 ? -0.0 : td));
    st_relaxed_u64(&scratch->partial[cid][1], (unsigned long long)__double_as_longlong(tp == 0.0 ? -0.0 : tp));
  }
  if (cid != 0) return;

  // Cluster 0's leader CTA folds: its 256 threads read all records at once (one L2 round trip when the other
  // clusters are done, which they are within a microsecond: the grid is one resident wave of equal shares),
  // re-reading the few that are still zero.  The wait is bounded: after RL_FOLD_LIMIT_NS without a record the
  // means are published as NaN, which no threshold comparison accepts.  The fold order is fixed (word index,
  // then a shuffle tree), so the result does not depend on arrival order at all.
  const unsigned words = 2 * (gridDim.x / csize);
  unsigned long long* flat = &scratch->partial[0][0];
  unsigned long long v[RL_FOLD_WORDS];
#pragma unroll
  for (int k = 0; k < RL_FOLD_WORDS; ++k) {
    const unsigned w = threadIdx.x + k * RL_THREADS;
    v[k] = w < words ? ld_relaxed_u64(flat + w) : 1ull;
  }
  bool timed_out = false;
  unsigned long long t0 = 0;
#pragma unroll
  for (int k = 0; k < RL_FOLD_WORDS; ++k) {
    const unsigned w = threadIdx.x + k * RL_THREADS;
    for (unsigned it = 0; v[k] == 0ull && !timed_out; ++it) {
      v[k] = ld_relaxed_u64(flat + w);
      if ((it & 63u) == 63u) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
        if (t0 == 0) t0 = now;
        else if (now - t0 > RL_FOLD_LIMIT_NS) timed_out = true;
      }
    }
  }
  // RL_THREADS is even, so a thread's words all have its own parity: even threads hold |prev - r| sums, odd
  // threads |prev| sums
  double acc = 0.0;
#pragma unroll
  for (int k = 0; k < RL_FOLD_WORDS; ++k) {
    const unsigned w = threadIdx.x + k * RL_THREADS;
    if (w < words) {
      acc += __longlong_as_double((long long)v[k]);
      st_relaxed_u64(flat + w, 0ull);  // leave the scratch zeroed for the next launch
    }
  }
#pragma unroll
  for (int o = 16; o >= 2; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);  // lanes of equal parity
  __shared__ double s_fold[RL_THREADS / 32][2];
  __shared__ int s_timeout;
  if (threadIdx.x == 0) s_timeout = 0;
  __syncthreads();
  if (lane < 2) s_fold[warp][lane] = acc;
  if (timed_out) s_timeout = 1;
  __syncthreads();
  if (threadIdx.x < 2) {
    double tot = 0.0;
#pragma unroll
    for (int i = 0; i < RL_THREADS / 32; ++i) tot += s_fold[i][threadIdx.x];
    const float mean = s_timeout ? __int_as_float(0x7fc00000) : A::round1((float)(tot / (double)n));
    means[threadIdx.x] = mean;
  }
}

// Cluster size of the reduction (CDB_RL_CLUSTER = 1, 2, 4 or 8; default RL_CLUSTER).
static int rel_l1_cluster() {
  static const int c = [] {
    const char* env = getenv("CDB_RL_CLUSTER");
    const int v = env ? atoi(env) : RL_CLUSTER;
    return (v == 1 || v == 2 || v == 4 || v == 8) ? v : RL_CLUSTER;
  }();
  return c;
}

template <class A, class A1, int U, bool HB, bool HP, bool WR>
static int launch_rel_l1_variant(const typename A::T* c, const typename A::T* b, const typename A::T* p,
                                 typename A::T* r, int64_t n, float* means, RelL1Scratch* scratch,
                                 cudaStream_t st) {
  auto kernel = rel_l1_kernel<A, A1, U, HB, HP, WR>;
  const int cluster = HP ? rel_l1_cluster() : 1;  // without a reduction there is nothing to share
  // the folding CTA waits for the other clusters' records, so the whole grid must be resident at once:
  // the wave is what the occupancy query promises, never more
  static PerDevice wave_of;
  const int64_t wave = wave_of.get([&] {
    return cluster > 1 ? resident_cluster_ctas(kernel, RL_THREADS, cluster) : resident_ctas(kernel, RL_THREADS);
  });
  const int64_t nchunk = n / (U * A::N);
  int64_t want = (nchunk + (int64_t)RL_THREADS * RL_UNROLL - 1) / ((int64_t)RL_THREADS * RL_UNROLL);
  int64_t cap = wave < (int64_t)RL_MAX_CLUSTERS * cluster ? wave : (int64_t)RL_MAX_CLUSTERS * cluster;
  int64_t grid = want < cap ? want : cap;
  grid = grid / cluster * cluster;
  if (grid < cluster) grid = cluster;
  CDB_CUDA_CHECK(launch_pdl_cluster(kernel, dim3((unsigned)grid), dim3(RL_THREADS), 0, st, (unsigned)cluster, c, b, p, r,
                                    n, means, scratch));
  return CDB_OK;
}

template <class A, class A1, int U>
static int launch_rel_l1(const void* cur, const void* base, const void* prev, void* res, int64_t n,
                         float* means, RelL1Scratch* scratch, cudaStream_t st) {
  using T = typename A::T;
  const T* c = static_cast<const T*>(cur);
  const T* b = static_cast<const T*>(base);
  const T* p = static_cast<const T*>(prev);
  T* r = static_cast<T*>(res);
#define CDB_RL(HB, HP, WR) return launch_rel_l1_variant<A, A1, U, HB, HP, WR>(c, b, p, r, n, means, scratch, st)
  const bool hb = base != nullptr, hp = prev != nullptr, wr = res != nullptr;
  if (hb && hp && wr) CDB_RL(true, true, true);
  else if (hb && hp && !wr) CDB_RL(true, true, false);
  else if (hb && !hp && wr) CDB_RL(true, false, true);
  else if (!hb && hp && wr) CDB_RL(false, true, true);
  else if (!hb && hp && !wr) CDB_RL(false, true, false);
  else if (!hb && !hp && wr) CDB_RL(false, false, true);
#undef CDB_RL
  return CDB_ERR_BAD_ARGUMENT;  // nothing to compute
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

template <class A, int U, int TERMS, bool ADD, bool EXACT>
__device__ __forceinline__ void apply_chunk(const typename A::T* hidden, const ApplyArgs& a,
                                            typename A::T* out, int64_t off) {
  using T = typename A::T;
  Chunk<A, U> h, o, d[TERMS];
  if constexpr (ADD) h = load_chunk<A, U>(hidden + off);
#pragma unroll
  for (int t = 0; t < TERMS; ++t) d[t] = load_chunk<A, U>(static_cast<const T*>(a.deriv[t]) + off);
#pragma unroll
  for (int i = 0; i < U; ++i) {
    // output = 0; output += (1/t!) * dY[t] * elapsed**t  -- three rounded ops per term
    typename A::V acc = A::zero();
#pragma unroll
    for (int t = 0; t < TERMS; ++t) {
      typename A::V term = A::template mulc<EXACT>(d[t].u[i], a.coef[t]);
      term = A::template mulc<EXACT>(term, a.power[t]);
      acc = A::add(acc, term);
    }
    if constexpr (ADD) acc = A::add(acc, h.u[i]);
    o.u[i] = acc;
  }
  store_chunk<A, U>(out + off, o);
}

template <class A, class A1, int U, int TERMS, bool ADD, bool EXACT>
__global__ void __launch_bounds__(EW_THREADS)
    taylor_apply_kernel(const typename A::T* __restrict__ hidden, const __grid_constant__ ApplyArgs a,
                        typename A::T* __restrict__ out, int64_t n) {
  constexpr int W = U * A::N;
  pdl_launch_dependents();
  pdl_wait_prior();
  const int64_t nchunk = n / W;
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
  for (; i + stride < nchunk; i += EW_UNROLL * stride) {
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u)
      apply_chunk<A, U, TERMS, ADD, EXACT>(hidden, a, out, (i + u * stride) * W);
  }
  if (i < nchunk) apply_chunk<A, U, TERMS, ADD, EXACT>(hidden, a, out, i * W);
  if constexpr (W > 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int64_t t = nchunk * W; t < n; ++t) apply_chunk<A1, 1, TERMS, ADD, false>(hidden, a, out, t);
  }
}

struct UpdateArgs {
  const void* prev[CDB_MAX_TAYLOR_TERMS];
  void* cur[CDB_MAX_TAYLOR_TERMS];
};

template <class A, int U, int NEW, bool HAS_BEFORE, bool WRITE_Y, bool POW2>
__device__ __forceinline__ void update_chunk(const typename A::T* after, const typename A::T* before,
                                             const UpdateArgs& a, float window, float inv_window,
                                             int64_t off) {
  using T = typename A::T;
  Chunk<A, U> y = load_chunk<A, U>(after + off);
  Chunk<A, U> b, p[NEW > 0 ? NEW : 1], o[NEW > 0 ? NEW : 1];
  if constexpr (HAS_BEFORE) b = load_chunk<A, U>(before + off);
#pragma unroll
  for (int k = 0; k < NEW; ++k) p[k] = load_chunk<A, U>(static_cast<const T*>(a.prev[k]) + off);
#pragma unroll
  for (int i = 0; i < U; ++i) {
    if constexpr (HAS_BEFORE) y.u[i] = A::sub(y.u[i], b.u[i]);  // Mn residual, rounded
    typename A::V v = y.u[i];
#pragma unroll
    for (int k = 0; k < NEW; ++k) {
      // dY[k+1] = (dY[k] - dY_prev[k]) / window : a rounded subtraction, then a rounded division
      v = A::template divc<POW2>(A::sub(v, p[k].u[i]), window, inv_window);
      o[k].u[i] = v;
    }
  }
  if constexpr (WRITE_Y) store_chunk<A, U>(static_cast<T*>(a.cur[0]) + off, y);
#pragma unroll
  for (int k = 0; k < NEW; ++k) store_chunk<A, U>(static_cast<T*>(a.cur[k + 1]) + off, o[k]);
}

template <class A, class A1, int U, int NEW, bool HAS_BEFORE, bool WRITE_Y, bool POW2>
__global__ void __launch_bounds__(EW_THREADS)
    taylor_update_kernel(const typename A::T* __restrict__ after, const typename A::T* __restrict__ before,
                         const __grid_constant__ UpdateArgs a, float window, float inv_window, int64_t n) {
  constexpr int W = U * A::N;
  pdl_launch_dependents();
  pdl_wait_prior();
  const int64_t nchunk = n / W;
  const int64_t stride = (int64_t)gridDim.x * EW_THREADS;
  int64_t i = (int64_t)blockIdx.x * EW_THREADS + threadIdx.x;
  for (; i + stride < nchunk; i += EW_UNROLL * stride) {
#pragma unroll
    for (int u = 0; u < EW_UNROLL; ++u)
      update_chunk<A, U, NEW, HAS_BEFORE, WRITE_Y, POW2>(after, before, a, window, inv_window,
                                                         (i + u * stride) * W);
  }
  if (i < nchunk)
    update_chunk<A, U, NEW, HAS_BEFORE, WRITE_Y, POW2>(after, before, a, window, inv_window, i * W);
  if constexpr (W > 1) {
    if (blockIdx.x == 0 && threadIdx.x == 0)
      for (int64_t t = nchunk * W; t < n; ++t)
        update_chunk<A1, 1, NEW, HAS_BEFORE, WRITE_Y, false>(after, before, a, window, inv_window, t);
  }
}

template <class A, class A1, int U, int TERMS, bool ADD, bool EX>
static void launch_apply_variant(const typename A::T* h, const ApplyArgs& a, typename A::T* o, int64_t n,
                                 cudaStream_t st) {
  auto kernel = taylor_apply_kernel<A, A1, U, TERMS, ADD, EX>;
  static PerDevice wave_of;
  const int64_t wave = wave_of.get([&] { return resident_ctas(kernel, EW_THREADS); });
  const int64_t nchunk = n / (U * A::N);
  int64_t want = (nchunk + (int64_t)EW_THREADS * EW_UNROLL - 1) / ((int64_t)EW_THREADS * EW_UNROLL);
  int64_t g = want < wave ? want : wave;
  (void)launch_pdl(kernel, dim3((unsigned)(g < 1 ? 1 : g)), dim3(EW_THREADS), 0, st, h, a, o, n);
}

template <class A, class A1, int U>
static int launch_apply(const void* hidden, const ApplyArgs& a, int n_terms, bool add, bool exact,
                        void* out, int64_t n, cudaStream_t st) {
  using T = typename A::T;
  const T* h = static_cast<const T*>(hidden);
  T* o = static_cast<T*>(out);
#define CDB_AP(TERMS)                                                                   \
  case TERMS:                                                                           \
    if (add && exact) launch_apply_variant<A, A1, U, TERMS, true, true>(h, a, o, n, st);  \
    else if (add) launch_apply_variant<A, A1, U, TERMS, true, false>(h, a, o, n, st);     \
    else if (exact) launch_apply_variant<A, A1, U, TERMS, false, true>(h, a, o, n, st);   \
    else launch_apply_variant<A, A1, U, TERMS, false, false>(h, a, o, n, st);             \
    break;
  switch (n_terms) {
    CDB_AP(1) CDB_AP(2) CDB_AP(3) CDB_AP(4) CDB_AP(5)
    default: return CDB_ERR_BAD_ARGUMENT;
  }
#undef CDB_AP
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

template <class A, class A1, int U, int NEW, bool HB, bool WY, bool P2>
static void launch_update_variant(const typename A::T* af, const typename A::T* bf, const UpdateArgs& a,
                                  float window, int64_t n, cudaStream_t st) {
  auto kernel = taylor_update_kernel<A, A1, U, NEW, HB, WY, P2>;
  static PerDevice wave_of;
  const int64_t wave = wave_of.get([&] { return resident_ctas(kernel, EW_THREADS); });
  const int64_t nchunk = n / (U * A::N);
  int64_t want = (nchunk + (int64_t)EW_THREADS * EW_UNROLL - 1) / ((int64_t)EW_THREADS * EW_UNROLL);
  int64_t g = want < wave ? want : wave;
  (void)launch_pdl(kernel, dim3((unsigned)(g < 1 ? 1 : g)), dim3(EW_THREADS), 0, st, af, bf, a, window, 1.0f / window, n);
}

template <class A, class A1, int U>
static int launch_update(const void* after, const void* before, const UpdateArgs& a, int n_new,
                         bool write_y, float window, bool pow2, int64_t n, cudaStream_t st) {
  using T = typename A::T;
  const T* af = static_cast<const T*>(after);
  const T* bf = static_cast<const T*>(before);
  const bool hb = before != nullptr;
#define CDB_UP2(NEW, HB, WY, P2) launch_update_variant<A, A1, U, NEW, HB, WY, P2>(af, bf, a, window, n, st)
#define CDB_UP(NEW)                                        \
  case NEW:                                                \
    if (hb && pow2) CDB_UP2(NEW, true, true, true);        \
    else if (hb) CDB_UP2(NEW, true, true, false);          \
    else if (write_y && pow2) CDB_UP2(NEW, false, true, true);   \
    else if (write_y) CDB_UP2(NEW, false, true, false);    \
    else if (pow2) CDB_UP2(NEW, false, false, true);       \
    else CDB_UP2(NEW, false, false, false);                \
    break;
  switch (n_new) {
    CDB_UP(0) CDB_UP(1) CDB_UP(2) CDB_UP(3) CDB_UP(4)
    default: return CDB_ERR_BAD_ARGUMENT;
  }
#undef CDB_UP
#undef CDB_UP2
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

// True when `c` survives a round trip through the storage type, i.e. the packed 16-bit multiply
// by the constant performs exactly the one rounding the float path would.
static bool representable(float c, int dtype) {
  if (dtype == CDB_F32) return true;
  if (dtype == CDB_BF16) return __bfloat162float(__float2bfloat16_rn(c)) == c;
  return __half2float(__float2half_rn(c)) == c && fabsf(c) <= 2048.f;
}
static bool is_pow2(float w) {
  int e = 0;
  return w > 0.f && frexpf(w, &e) == 0.5f && e >= -20 && e <= 20;
}

}  // namespace cdb

// ------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------
using namespace cdb;

#define CDB_DISPATCH(FN, vec, ...)                                                                  \
  switch (dtype) {                                                                                  \
    case CDB_F32:                                                                                   \
      return vec ? FN<F32x1, F32x1, 4>(__VA_ARGS__) : FN<F32x1, F32x1, 1>(__VA_ARGS__);              \
    case CDB_BF16:                                                                                  \
      return vec ? FN<BF16x2, BF16x1, 4>(__VA_ARGS__) : FN<BF16x1, BF16x1, 1>(__VA_ARGS__);          \
    case CDB_F16:                                                                                   \
      return vec ? FN<F16x2, F16x1, 4>(__VA_ARGS__) : FN<F16x1, F16x1, 1>(__VA_ARGS__);              \
    default:                                                                                        \
      return CDB_ERR_BAD_ARGUMENT;                                                                  \
  }

extern "C" size_t cdb_rel_l1_scratch_bytes(void) { return sizeof(RelL1Scratch); }

extern "C" int cdb_rel_l1(const void* cur, const void* base, const void* prev, void* residual_out,
                          int64_t n, int dtype, float* means, void* scratch, size_t scratch_bytes,
                          void* stream) {
  if (!cur || n <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (!prev && !residual_out) return CDB_ERR_BAD_ARGUMENT;
  if (prev && (!means || !scratch)) return CDB_ERR_BAD_ARGUMENT;
  if (prev && scratch_bytes < sizeof(RelL1Scratch)) return CDB_ERR_SCRATCH_TOO_SMALL;
  if (prev && (reinterpret_cast<uintptr_t>(scratch) & 127u)) return CDB_ERR_UNSUPPORTED;
  if (residual_out && !base && residual_out == cur) residual_out = nullptr;  // nothing to copy
  if (!prev && !residual_out) return CDB_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  RelL1Scratch* sc = static_cast<RelL1Scratch*>(scratch);
  const bool vec = aligned16(cur) && aligned16(base) && aligned16(prev) && aligned16(residual_out);
  CDB_DISPATCH(launch_rel_l1, vec, cur, base, prev, residual_out, n, means, sc, st)
}

extern "C" int cdb_taylor_apply(const void* hidden, const void* const* derivs, const float* coef,
                                const float* power, int n_terms, int add_hidden, void* out,
                                int64_t n, int dtype, void* stream) {
  if (!derivs || !coef || !power || !out || n <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (n_terms < 1 || n_terms > CDB_MAX_TAYLOR_TERMS) return CDB_ERR_BAD_ARGUMENT;
  if (add_hidden && !hidden) return CDB_ERR_BAD_ARGUMENT;
  ApplyArgs a{};
  bool vec = aligned16(out) && (!add_hidden || aligned16(hidden));
  bool exact = true;
  for (int t = 0; t < n_terms; ++t) {
    if (!derivs[t]) return CDB_ERR_BAD_ARGUMENT;
    a.deriv[t] = derivs[t];
    a.coef[t] = coef[t];
    a.power[t] = power[t];
    vec = vec && aligned16(derivs[t]);
    exact = exact && representable(coef[t], dtype) && representable(power[t], dtype);
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool add = add_hidden != 0;
  CDB_DISPATCH(launch_apply, vec, hidden, a, n_terms, add, exact, out, n, st)
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
  if (n_new == 0) window = 1.f;
  const bool pow2 = is_pow2(window);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  CDB_DISPATCH(launch_update, vec, after, before, a, n_new, write_y, window, pow2, n, st)
}

// ------------------------------------------------------------------------------------------
// Relative-L1 check for callers that cannot allocate device memory
// ------------------------------------------------------------------------------------------
// Some hosts of this library are not allowed to call cudaMalloc (or anything that does it for
// them) around the check: a plug-in running inside another framework's memory pool, a process
// whose device memory is fully pre-partitioned, a serving loop with a "no allocation after
// warm-up" rule.  cdb_rel_l1 asks such a caller for a scratch buffer it has no clean way to
// provide.  This variant brings its own: the reduction scratch lives in the library's image as a
// file-scope device array, so every device that loads the library holds these bytes until the
// process exits, and no allocation is made at any point.
static __device__ __align__(256) unsigned char g_rel_l1_static_scratch[sizeof(cdb::RelL1Scratch)];

namespace cdb {

// Host code may not hand `g_rel_l1_static_scratch` to a kernel: on the host that name is only a
// stand-in for the symbol.  Its device address is looked up once per device (with that device
// current) and cached.
static int static_scratch_for_current_device(RelL1Scratch** out) {
  constexpr int kMaxDevices = 64;
  static RelL1Scratch* cached[kMaxDevices] = {};
  static std::mutex mu;
  int dev = -1;
  CDB_CUDA_CHECK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return CDB_ERR_UNSUPPORTED;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    CDB_CUDA_CHECK(cudaGetSymbolAddress(&p, g_rel_l1_static_scratch));
    if (p == nullptr) return CDB_ERR_CUDA;
    cached[dev] = static_cast<RelL1Scratch*>(p);
  }
  *out = cached[dev];
  return CDB_OK;
}

}  // namespace cdb

extern "C" int cdb_rel_l1_static(const void* cur, const void* base, const void* prev, void* residual_out,
                                 int64_t n, int dtype, float* means, void* stream) {
  if (!cur || !prev || !means || n <= 0) return CDB_ERR_BAD_ARGUMENT;
  if (n > CDB_REL_L1_STATIC_MAX_ELEMS) {
    cdb::set_error_text("cdb_rel_l1_static: n exceeds CDB_REL_L1_STATIC_MAX_ELEMS (2^30 elements); "
                        "use cdb_rel_l1 with caller-provided scratch for larger tensors");
    return CDB_ERR_TOO_LARGE;
  }
  // The array's address is per device and is looked up for the CURRENT device, so the tensors must live
  // there too: with another device current the kernel would be handed that device's copy of the array.
  cudaPointerAttributes attr{};
  int cur_dev = -1;
  CDB_CUDA_CHECK(cudaGetDevice(&cur_dev));
  if (cudaPointerGetAttributes(&attr, cur) != cudaSuccess || attr.type != cudaMemoryTypeDevice ||
      attr.device != cur_dev) {
    (void)cudaGetLastError();
    cdb::set_error_text("cdb_rel_l1_static: `cur` is not device memory of the current device; make the "
                        "device that owns the tensors current before the call");
    return CDB_ERR_BAD_ARGUMENT;
  }
  RelL1Scratch* sc = nullptr;
  int rc = static_scratch_for_current_device(&sc);
  if (rc != CDB_OK) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The array is shared by every call and keeps whatever the previous call left in it.  Only the
  // arrival counter and the two accumulators have to start at zero; clear them on the caller's
  // stream so a launch that was cut short earlier cannot poison this one.
  CDB_CUDA_CHECK(cudaMemsetAsync(sc, 0, sizeof(RelL1Scratch), st));
  if (residual_out && !base && residual_out == cur) residual_out = nullptr;
  const bool vec = aligned16(cur) && aligned16(base) && aligned16(prev) && aligned16(residual_out);
  CDB_DISPATCH(launch_rel_l1, vec, cur, base, prev, residual_out, n, means, sc, st)
}
