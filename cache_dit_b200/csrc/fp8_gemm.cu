// Row-scaled FP8 (e4m3) GEMM for sm_100a: out[m,n] = (sum_k A[m,k] W[n,k]) * sa[m] * sw[n] (+ bias[n])
//
// Blackwell-native structure
//   * operands: TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) into a shared-memory ring of 4 to 8 stages
//     (192 KB; 6 stages of 32 KB in the CTA-pair kernel), one CTA per SM, every CTA loads its own tiles (no
//     cluster-wide loads);
//   * math: tcgen05.mma.kind::f8f6f4 issued by one elected thread, fp32 accumulators in tensor memory (TMEM):
//     cta_group::1, 128 x bn x 32 per instruction (bn a multiple of 16 up to 256) in the single-CTA kernel,
//     cta_group::2, 256 x 256 x 32 over a pair of SMs in the CTA-pair kernel further down;
//   * an optional tanh-GELU of output columns in the epilogue (the MLP-in projection of a transformer block);
//   * two 256-column TMEM accumulators so the epilogue of tile i overlaps the main loop of tile i+1;
//   * epilogue: tcgen05.ld (32 lanes x 32 columns per warp), per-row x per-column scale, optional
//     bias, bf16 pack into a swizzled shared-memory staging block, TMA store (cp.async.bulk.tensor
//     shared -> global) of 32 x 64 blocks: whole 128-byte lines leave the SM, instead of one
//     16-byte piece per thread and row, which kept the L1 data path as busy as the operand loads;
//   * persistent grid (one CTA per SM), static tile order: M fastest inside groups of 16 row tiles, so
//     the CTAs of a wave share weight tiles and a bounded set of A panels in L2.
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA issuer,
// warps 2..5 = epilogue (TMEM lane quarter = warp % 4).
//
// Every mbarrier wait is bounded: after ~2 s without progress the waiter raises a CTA-wide abort
// flag, records a code in the caller's status word, all roles drain, TMEM is released and the
// kernel returns, so a logic error cannot wedge the device.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <utility>
#include <unordered_map>

#include "common.cuh"

namespace cdb {

constexpr int BM = 128;          // tile rows   (UMMA M)
constexpr int BN = 256;          // tile cols   (UMMA N)
constexpr int BK = 128;          // K bytes per stage = one 128-byte swizzle span of e4m3
constexpr int UMMA_K = 32;       // K per tcgen05.mma for 8-bit inputs
constexpr int STAGES = 4;        // stages of the ring at the full tile width
constexpr int MAX_STAGES = 8;    // narrower tiles have smaller stages: more of them fit the same ring
constexpr int GEMM_THREADS = 192;
constexpr int EPI_WARP0 = 2;
constexpr int EPI_THREADS = 128;
constexpr uint32_t TMEM_COLS = 512;  // 2 accumulators x 256 fp32 columns
constexpr int A_STAGE_BYTES = BM * BK;
constexpr int B_STAGE_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;
// Which kernel large-M problems use unless CDB_GEMM_KERNEL overrides it.
#ifndef CDB_GEMM_DEFAULT_PAIR
#define CDB_GEMM_DEFAULT_PAIR 1
#endif

struct __align__(8) GemmBarriers {
  uint64_t full[MAX_STAGES];   // TMA bytes landed
  uint64_t empty[MAX_STAGES];  // MMAs reading the stage retired
  uint64_t acc_full[2];        // accumulator complete in TMEM
  uint64_t acc_empty[2];       // epilogue drained the accumulator
  uint32_t tmem_base;
  volatile int abort_flag;
};

// Epilogue staging: per epilogue warp two blocks of 32 rows x 64 bf16 columns (128-byte rows,
// 128-byte swizzle, what the output tensor map's box expects).
constexpr int OUT_BOX_COLS = 64;
constexpr int OUT_BOX_ROWS = 32;
constexpr int OUT_BLOCK_BYTES = OUT_BOX_ROWS * OUT_BOX_COLS * 2;  // 4096
constexpr int OUT_STAGING_BYTES = (EPI_THREADS / 32) * 2 * OUT_BLOCK_BYTES;

// dynamic shared memory:
// [<=1023 B alignment slack][STAGES x (A tile | B tile)][output staging][col scale f32][bias bf16][barriers]
constexpr int SMEM_TILE_BYTES = STAGES * STAGE_BYTES;
constexpr int SMEM_EXTRA_BYTES = OUT_STAGING_BYTES + BN * 4 + BN * 2 + (int)sizeof(GemmBarriers);
constexpr int SMEM_TOTAL_BYTES = 1024 + SMEM_TILE_BYTES + SMEM_EXTRA_BYTES;
static_assert(SMEM_TOTAL_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");

// ---- PTX wrappers ------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait. Returns false if the CTA is aborting (or the wait itself ran out).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, GemmBarriers* gb,
                                          int32_t* status_word, int code) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (gb->abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) {
        gb->abort_flag = 1;
        if (status_word) atomicCAS(status_word, 0, code);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(const CUtensorMap* map, uint64_t* bar, void* dst, int c0,
                                            int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tcgen05_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tcgen05_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]),
        "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]),
        "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]),
        "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major tile stored as rows of 128 bytes with the
// 128-byte swizzle (exactly what the TMA box writes): 8-row groups are 1024 bytes apart.
//   bits [0,14)  start address >> 4        bits [16,30) leading byte offset >> 4 (unused: 1)
//   bits [32,46) stride byte offset >> 4   bits [46,48) descriptor version = 1
//   bits [61,64) layout type = 2 (128-byte swizzle)
__device__ __forceinline__ uint64_t make_kmajor_sw128_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// Instruction descriptor, kind::f8f6f4: D = fp32, A = B = e4m3, both K-major, dense.
//   bits [4,6) D format (1 = f32)   [7,10) A format (0 = e4m3)   [10,13) B format (0 = e4m3)
//   bit 15 / 16 A / B major (0 = K) [17,23) N >> 3               [24,29) M >> 4
constexpr uint32_t idesc_e4m3_f32(int m, int n) {
  return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// AND-reduction of a predicate over the 128 epilogue threads (named barrier 1).
__device__ __forceinline__ bool epi_all(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t.reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.and.pred q, 1, %2, p;\n\t"
      "selp.u32 %0, 1, 0, q;\n\t}"
      : "=r"(r)
      : "r"((uint32_t)pred), "n"(EPI_THREADS)
      : "memory");
  return r != 0;
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// TMA store of one staged block: shared (this CTA) -> global through the output tensor map.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* src, int c0, int c1) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
               "r"(smem_u32(src)), "r"(c0), "r"(c1)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// Wait until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_group_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// One epilogue warp's share of a tile: 32 accumulator rows (TMEM lanes) x `bn` columns.  Per block of
// 64 columns: two tcgen05.ld, scale + bias, bf16 pack, 16-byte shared stores at the 128-byte-swizzled
// position (chunk ^ (row % 8)): conflict-free, then one TMA store.  The tensor map clips rows >= M
// and columns >= N.  `blocks_done` counts this warp's stores so the two staging blocks alternate.
// A tile width that is not a multiple of 64 leaves a last block of 16, 32 or 48 columns: a 64-column TMA
// store would spill into the neighbouring tile's columns, so that block goes out as 16-byte global stores
// straight from the registers.
// tanh-GELU of an output pair that has already been rounded to bf16, rounded to bf16 again: what an eager
// `gelu(linear(x))` computes, and bit for bit what the GELU variant of the quantization kernel computes when it
// reads the linear's output back.
__device__ __forceinline__ uint32_t gelu_bf16x2(uint32_t w) {
  return pack_bf16x2(gelu_tanh(__uint_as_float(w << 16)), gelu_tanh(__uint_as_float(w & 0xffff0000u)));
}
__device__ __forceinline__ void epilogue_rows(const CUtensorMap* map_out, __nv_bfloat16* out, int64_t ld_out,
                                              uint8_t* staging, uint32_t taddr, float rs,
                                              const float* s_colscale, const __nv_bfloat16* s_bias, int row0,
                                              int n0, int M, int N, int bn, int act_col, int lane,
                                              uint32_t& blocks_done) {
  if (row0 >= M) return;  // the whole 32-row slice is padding
#pragma unroll 1
  for (int cblk = 0; cblk < bn; cblk += OUT_BOX_COLS) {
    if (n0 + cblk >= N) break;
    const int valid = min(OUT_BOX_COLS, bn - cblk);  // warp-uniform
    uint32_t acc[2][32];
    tmem_ld_32x32b_x32(taddr + cblk, acc[0]);
    if (valid > 32) tmem_ld_32x32b_x32(taddr + cblk + 32, acc[1]);
    if (valid < OUT_BOX_COLS) {
      tmem_ld_wait();
      const int row = row0 + lane;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int cb = cblk + h * 32 + g * 8;
          if (h * 32 + g * 8 < valid && n0 + cb < N && row < M) {
            uint32_t w[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int c = cb + 2 * j;
              const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(s_bias + c));
              const float v0 = __uint_as_float(acc[h][g * 8 + 2 * j]) * rs * s_colscale[c] + b.x;
              const float v1 = __uint_as_float(acc[h][g * 8 + 2 * j + 1]) * rs * s_colscale[c + 1] + b.y;
              w[j] = pack_bf16x2(v0, v1);
              if (n0 + cb >= act_col) w[j] = gelu_bf16x2(w[j]);
            }
            *reinterpret_cast<uint4*>(out + (int64_t)row * ld_out + n0 + cb) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      continue;
    }
    uint8_t* block = staging + (blocks_done & 1u) * OUT_BLOCK_BYTES;
    if (lane == 0) bulk_wait_group_read<1>();  // the store that used this block two blocks ago is done reading
    __syncwarp();
    tmem_ld_wait();
    uint8_t* rowp = block + lane * (OUT_BOX_COLS * 2);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
#pragma unroll
      for (int g = 0; g < 4; ++g) {  // 8 columns = one 16-byte chunk
        const int cb = cblk + h * 32 + g * 8;
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c = cb + 2 * j;
          const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(s_bias + c));
          const float v0 = __uint_as_float(acc[h][g * 8 + 2 * j]) * rs * s_colscale[c] + b.x;
          const float v1 = __uint_as_float(acc[h][g * 8 + 2 * j + 1]) * rs * s_colscale[c + 1] + b.y;
          w[j] = pack_bf16x2(v0, v1);
        }
        if (n0 + cb >= act_col) {  // warp-uniform: act_col is a multiple of 8
#pragma unroll
          for (int j = 0; j < 4; ++j) w[j] = gelu_bf16x2(w[j]);
        }
        const int chunk = (h * 4 + g) ^ (lane & 7);
        *reinterpret_cast<uint4*>(rowp + chunk * 16) = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    fence_async_smem();  // make the generic-proxy writes visible to the bulk-copy engine
    __syncwarp();
    if (lane == 0) {
      tma_store_2d(map_out, block, n0 + cblk, row0);
      bulk_commit_group();
    }
    ++blocks_done;
  }
}

// One launch can run two independent products (a "problem set"): the second is meant to be small (the
// text stream of a double-stream block beside the image stream's product of the same layer) and its
// tiles come last, so they fill the SMs the first problem's final, partial wave leaves idle instead of
// paying a launch, a pipeline start and a mostly empty grid of their own.
constexpr int MAX_PROBLEMS = 2;
struct GemmProblem {
  CUtensorMap map_a, map_w, map_out;
  const float* sa;
  const float* sw;
  const __nv_bfloat16* bias;
  __nv_bfloat16* out;  // for the ragged last column block of a tile (see epilogue_rows)
  int64_t ld_out;
  int M, N, K;
  int m_tiles, n_tiles, k_blocks, group_m;
  int tile_begin;  // index of this problem's first tile in the launch's tile sequence
  int act_col;     // output columns >= act_col pass through tanh-GELU in the epilogue (INT32_MAX: none)
  // Tile width in columns: a multiple of 16 up to BN, chosen on the host so that the tile count fills whole
  // waves of SMs (the CTA-pair kernel: BN unless a multiple of 32 is forced).  `idesc` is the instruction
  // descriptor for that width.
  int bn;
  uint32_t idesc;
};
struct GemmProblems {
  GemmProblem p[MAX_PROBLEMS];
  int count;
  int num_tiles;
  int stages;       // single-CTA kernel: stages of the shared-memory ring for this launch's tile width
  int stage_bytes;  // ... and the size of one (A tile | weight tile) stage
};
__device__ __forceinline__ const GemmProblem* problem_of(const GemmProblems& ps, int tile, int& local) {
  const bool second = ps.count > 1 && tile >= ps.p[1].tile_begin;
  const GemmProblem* pr = second ? &ps.p[1] : &ps.p[0];
  local = tile - pr->tile_begin;
  return pr;
}

// Tile order: M fastest inside groups of `group_m` row tiles, all column tiles of a group before
// the next group.  The CTAs of a wave then share a few weight tiles AND at most TILE_GROUP_M row
// panels of A, so both operands are re-read from L2; with plain M-fastest order an A that does not fit
// the L2 (M = 16384, K = 12288: 201 MB) was streamed from HBM once per column tile.
// The group size is chosen on the host (tile_group_rows): all row tiles when there are few (every weight
// tile is then read from HBM once), else balanced groups of at most 16.
__device__ __forceinline__ void tile_coords(int tile, int m_tiles, int n_tiles, int group_m, int& mi, int& ni) {
  const int per_group = group_m * n_tiles;
  const int group = tile / per_group;
  const int first_m = group * group_m;
  const int rows = min(group_m, m_tiles - first_m);  // the last group may be short
  const int in_group = tile - group * per_group;
  mi = first_m + in_group % rows;
  ni = in_group / rows;
}

// ---- kernel --------------------------------------------------------------------------------
__global__ void __launch_bounds__(GEMM_THREADS, 1)
    fp8_gemm_rowscaled_kernel(const __grid_constant__ GemmProblems ps, int32_t* status_word) {
  extern __shared__ uint8_t smem_raw[];
  // 128-byte swizzle needs 1024-byte aligned tiles.
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* s_staging = smem + SMEM_TILE_BYTES;  // 1024-byte aligned: the tile ring is a multiple of 1024
  float* s_colscale = reinterpret_cast<float*>(s_staging + OUT_STAGING_BYTES);
  __nv_bfloat16* s_bias = reinterpret_cast<__nv_bfloat16*>(s_colscale + BN);
  GemmBarriers* gb = reinterpret_cast<GemmBarriers*>(s_bias + BN);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = ps.num_tiles;
  pdl_launch_dependents();  // a following kernel launched as a programmatic dependent may be scheduled early

  if (threadIdx.x == 0) {
    for (int s = 0; s < MAX_STAGES; ++s) {
      mbar_init(&gb->full[s], 1);
      mbar_init(&gb->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&gb->acc_full[b], 1);
      mbar_init(&gb->acc_empty[b], EPI_THREADS / 32);
    }
    gb->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&gb->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  tcgen05_fence_after();
  const uint32_t tmem_base = gb->tmem_base;

  const int stages = ps.stages;
  const int stage_bytes = ps.stage_bytes;
  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      for (int i = 0; i < ps.count; ++i) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&ps.p[i].map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&ps.p[i].map_w) : "memory");
      }
    }
    uint32_t it = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int local;
      const GemmProblem* pr = problem_of(ps, tile, local);
      const int k_blocks = pr->k_blocks;
      int mi, ni;
      tile_coords(local, pr->m_tiles, pr->n_tiles, pr->group_m, mi, ni);
      const int m0 = mi * BM, n0 = ni * pr->bn;
      const uint32_t stage_tx = A_STAGE_BYTES + (uint32_t)pr->bn * BK;  // the weight box has `bn` rows
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        if (lane == 0) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          ok = mbar_wait(&gb->empty[s], ph ^ 1u, gb, status_word, 1);
          if (ok) {
            uint8_t* a_dst = smem + s * stage_bytes;
            uint8_t* b_dst = a_dst + A_STAGE_BYTES;
            mbar_expect_tx(&gb->full[s], stage_tx);
            tma_load_2d(&pr->map_a, &gb->full[s], a_dst, kb * BK, m0);
            tma_load_2d(&pr->map_w, &gb->full[s], b_dst, kb * BK, n0);
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
      }
    }
    if (lane == 0) {
      // Do not let the CTA retire while bulk copies into its shared memory are in flight:
      // wait (bounded) until every armed stage has landed.
      const uint32_t issued = it;
      for (uint32_t j = (issued > (uint32_t)stages ? issued - stages : 0); j < issued; ++j) {
        const int s = j % stages;
        const uint32_t ph = (j / stages) & 1u;
        uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(&gb->full[s], ph)) {
          if (global_timer_ns() - t0 > WAIT_LIMIT_NS) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
        const uint32_t buf = local_tile & 1u;
        const uint32_t use = local_tile >> 1;  // how many times this buffer was used before
        ok = mbar_wait(&gb->acc_empty[buf], (use & 1u) ^ 1u, gb, status_word, 2);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        int local;
        const GemmProblem* pr = problem_of(ps, tile, local);
        const int k_blocks = pr->k_blocks;
        const uint32_t idesc = pr->idesc;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % stages;
          const uint32_t ph = (it / stages) & 1u;
          ok = mbar_wait(&gb->full[s], ph, gb, status_word, 3);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * stage_bytes);
          const uint32_t b_addr = a_addr + A_STAGE_BYTES;
          const uint64_t adesc = make_kmajor_sw128_desc(a_addr);
          const uint64_t bdesc = make_kmajor_sw128_desc(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // advance 32 bytes along K inside the swizzle span: +2 in the (addr >> 4) field
            umma_f8(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)),
                    idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tcgen05_commit(&gb->empty[s]);  // frees the stage once these MMAs retire
        }
        if (ok) tcgen05_commit(&gb->acc_full[buf]);
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int quarter = warp & 3;            // TMEM lanes [32*quarter, 32*quarter + 32)
    const int et = threadIdx.x - EPI_WARP0 * 32;  // 0..127
    uint32_t local_tile = 0, blocks_done = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local_tile) {
      int local;
      const GemmProblem* pr = problem_of(ps, tile, local);
      const int M = pr->M, N = pr->N;
      const float* sa = pr->sa;
      const float* sw = pr->sw;
      const __nv_bfloat16* bias = pr->bias;
      int mi, ni;
      tile_coords(local, pr->m_tiles, pr->n_tiles, pr->group_m, mi, ni);
      const int bn = pr->bn;
      const int m0 = mi * BM, n0 = ni * bn;
      const uint32_t buf = local_tile & 1u;
      const uint32_t use = local_tile >> 1;
      // (1) the previous tile's readers of the staged column scales are done
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      for (int c = et; c < bn; c += EPI_THREADS) {
        const int col = n0 + c;
        s_colscale[c] = col < N ? __ldg(sw + col) : 0.f;
        s_bias[c] = (bias != nullptr && col < N) ? bias[col] : __float2bfloat16(0.f);
      }
      ok = mbar_wait(&gb->acc_full[buf], use & 1u, gb, status_word, 4);
      // (2) one barrier publishes the staged scales AND makes the continue/abort decision uniform
      // over the four epilogue warps, so no warp can be left alone at barrier (1).
      ok = epi_all(ok);
      if (!ok) break;
      tcgen05_fence_after();

      const int row = m0 + quarter * 32 + lane;
      const float rs = row < M ? __ldg(sa + row) : 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      epilogue_rows(&pr->map_out, pr->out, pr->ld_out, s_staging + quarter * 2 * OUT_BLOCK_BYTES, taddr, rs,
                    s_colscale, s_bias, m0 + quarter * 32, n0, M, N, bn, pr->act_col, lane, blocks_done);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&gb->acc_empty[buf]);
    }
    if (lane == 0) bulk_wait_group_all();  // staged blocks are read and written out before the CTA retires
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---- CTA-pair variant (tcgen05 cta_group::2) ---------------------------------------------------
// Two CTAs on the two SMs of a TPC work on one 256 x 256 tile.  Each CTA loads its own 128 rows
// of A and only HALF of the weight tile (128 of its 256 rows); one elected thread of the even CTA
// issues a single 256 x 256 x 32 MMA per K step that reads both halves through the pair's shared
// memory, and each CTA receives the accumulator rows of its own A half in its own TMEM.  Per flop
// this moves 2/3 of the bytes from L2 into shared memory and half of the weight bytes per SM,
// which is what limits the single-CTA kernel.  No data is multicast anywhere: every TMA copy is a
// plain per-CTA load whose completion is counted on the even CTA's barrier.  The MMA's completion is
// committed to the same barrier of both CTAs by one commit whose ARRIVAL is multicast to the pair.
constexpr int P_STAGES = 6;
constexpr int P_A_BYTES = 128 * BK;  // 128 rows of A per CTA
constexpr int P_B_BYTES = 128 * BK;  // 128 rows (half) of the weight tile per CTA
constexpr int P_STAGE_BYTES = P_A_BYTES + P_B_BYTES;
constexpr int P_BM = 256;            // tile rows per CTA pair

struct __align__(8) PairBarriers {
  uint64_t full[P_STAGES];   // even CTA's copy is used: bytes of both CTAs land here
  uint64_t empty[P_STAGES];  // per CTA: the MMAs that read this CTA's stage have retired
  uint64_t acc_full[2];      // per CTA: accumulator complete
  uint64_t acc_empty[2];     // even CTA's copy is used: both CTAs' epilogues drained the buffer
  uint32_t tmem_base;
  volatile int abort_flag;
};
constexpr int P_SMEM_TILE_BYTES = P_STAGES * P_STAGE_BYTES;
constexpr int P_SMEM_TOTAL_BYTES =
    1024 + P_SMEM_TILE_BYTES + OUT_STAGING_BYTES + BN * 4 + BN * 2 + (int)sizeof(PairBarriers);
static_assert(P_SMEM_TOTAL_BYTES <= 232448, "exceeds the 227 KB of shared memory a CTA can opt in to");

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of the same shared-memory location in the CTA with the given rank of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// Per-CTA TMA load of a CTA pair: data goes to this CTA's shared memory, the byte count is
// reported to the barrier at `bar_cluster_addr` (the even CTA's).
__device__ __forceinline__ void tma_load_2d_pair(const CUtensorMap* map, uint32_t bar_cluster_addr, void* dst,
                                                 int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void umma_f8_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                             uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive, when all MMAs issued so far retire, on the barrier at this shared-memory offset in BOTH CTAs of the pair
// with one instruction (a commit sits in the MMA issue stream: one per K block instead of two measured 4-8 %
// on a load-free run of this kernel).  Multicast of a barrier arrival only: no data moves.
__device__ __forceinline__ void tcgen05_commit_both(uint32_t bar_cta_addr) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
          bar_cta_addr),
      "h"((uint16_t)3)
      : "memory");
}
__device__ __forceinline__ bool pair_wait(uint64_t* bar, uint32_t parity, PairBarriers* gb, int32_t* status_word,
                                          int code) {
  uint64_t t0 = 0;
  for (uint32_t it = 0;; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((it & 255u) == 255u) {
      if (gb->abort_flag) return false;
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > WAIT_LIMIT_NS) {
        gb->abort_flag = 1;
        if (status_word) atomicCAS(status_word, 0, code);
        return false;
      }
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
    fp8_gemm_rowscaled_pair_kernel(const __grid_constant__ GemmProblems ps, int32_t* status_word) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* s_staging = smem + P_SMEM_TILE_BYTES;
  float* s_colscale = reinterpret_cast<float*>(s_staging + OUT_STAGING_BYTES);
  __nv_bfloat16* s_bias = reinterpret_cast<__nv_bfloat16*>(s_colscale + BN);
  PairBarriers* gb = reinterpret_cast<PairBarriers*>(s_bias + BN);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();  // 0 = even CTA: owns the shared barriers, issues the MMAs
  const int num_tiles = ps.num_tiles;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;
  pdl_launch_dependents();  // a following kernel launched as a programmatic dependent may be scheduled early

  if (threadIdx.x == 0) {
    for (int s = 0; s < P_STAGES; ++s) {
      mbar_init(&gb->full[s], 1);
      mbar_init(&gb->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&gb->acc_full[b], 1);
      mbar_init(&gb->acc_empty[b], 2 * (EPI_THREADS / 32));
    }
    gb->abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {  // the same warp of both CTAs allocates the pair's tensor memory
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(&gb->tmem_base)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // the peer's barriers exist before anything is signalled across the pair
  tcgen05_fence_after();
  const uint32_t tmem_base = gb->tmem_base;

  if (warp == 0) {
    // ---------------- TMA producer (both CTAs) ----------------
    if (lane == 0) {
      for (int i = 0; i < ps.count; ++i) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&ps.p[i].map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&ps.p[i].map_w) : "memory");
      }
    }
    const int half = (int)rank * 128;  // this CTA's rows of A and its half of the weight tile
    uint32_t it = 0;
    bool ok = true;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs) {
      int local;
      const GemmProblem* pr = problem_of(ps, tile, local);
      const int k_blocks = pr->k_blocks;
      int mi, ni;
      tile_coords(local, pr->m_tiles, pr->n_tiles, pr->group_m, mi, ni);
      const int m0 = mi * P_BM + half;
      const int n0 = ni * pr->bn + (int)rank * (pr->bn >> 1);  // this CTA's half of the weight tile
      const uint32_t pair_tx = 2u * (uint32_t)(P_A_BYTES + (pr->bn >> 1) * BK);  // both CTAs' bytes of one stage
      for (int kb = 0; kb < k_blocks; ++kb, ++it) {
        if (lane == 0) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          ok = pair_wait(&gb->empty[s], ph ^ 1u, gb, status_word, 11);
          if (ok) {
            uint8_t* a_dst = smem + s * P_STAGE_BYTES;
            uint8_t* b_dst = a_dst + P_A_BYTES;
            if (rank == 0) mbar_expect_tx(&gb->full[s], pair_tx);
            const uint32_t full_addr = map_to_cta(smem_u32(&gb->full[s]), 0);
            tma_load_2d_pair(&pr->map_a, full_addr, a_dst, kb * BK, m0);
            tma_load_2d_pair(&pr->map_w, full_addr, b_dst, kb * BK, n0);
          }
        }
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        if (!ok) break;
      }
    }
    if (lane == 0) {
      // A CTA may not retire while copies into its shared memory are in flight or while the peer's
      // MMAs still read its tiles: wait (bounded) until the consumer has released every stage used.
      const uint32_t issued = it;
      for (uint32_t j = (issued > P_STAGES ? issued - P_STAGES : 0); j < issued; ++j) {
        const int s = j % P_STAGES;
        const uint32_t ph = (j / P_STAGES) & 1u;
        uint64_t t0 = global_timer_ns();
        while (!mbar_try_wait(&gb->empty[s], ph)) {
          if (gb->abort_flag || global_timer_ns() - t0 > WAIT_LIMIT_NS) break;
        }
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ---------------- MMA issuer (even CTA only) ----------------
    if (lane == 0 && rank == 0) {
      uint32_t it = 0, local_tile = 0;
      bool ok = true;
      for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
        const uint32_t buf = local_tile & 1u;
        const uint32_t use = local_tile >> 1;
        ok = pair_wait(&gb->acc_empty[buf], (use & 1u) ^ 1u, gb, status_word, 12);
        if (!ok) break;
        tcgen05_fence_after();
        const uint32_t tmem_d = tmem_base + buf * BN;
        int local;
        const GemmProblem* pr = problem_of(ps, tile, local);
        const int k_blocks = pr->k_blocks;
        const uint32_t idesc = pr->idesc;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % P_STAGES;
          const uint32_t ph = (it / P_STAGES) & 1u;
          ok = pair_wait(&gb->full[s], ph, gb, status_word, 13);
          if (!ok) break;
          tcgen05_fence_after();
          const uint32_t a_addr = smem_u32(smem + s * P_STAGE_BYTES);
          const uint64_t adesc = make_kmajor_sw128_desc(a_addr);
          const uint64_t bdesc = make_kmajor_sw128_desc(a_addr + P_A_BYTES);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            umma_f8_pair(tmem_d, adesc + (uint64_t)(k * (UMMA_K >> 4)), bdesc + (uint64_t)(k * (UMMA_K >> 4)),
                         idesc, (kb | k) != 0 ? 1u : 0u);
          }
          tcgen05_commit_both(smem_u32(&gb->empty[s]));  // frees the stage in this CTA and in the peer
        }
        if (ok) {
          tcgen05_commit_both(smem_u32(&gb->acc_full[buf]));
        }
      }
    }
    __syncwarp();
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs): this CTA's 128 rows x 256 columns ----------------
    const int quarter = warp & 3;
    const int et = threadIdx.x - EPI_WARP0 * 32;
    uint32_t local_tile = 0, blocks_done = 0;
    bool ok = true;
    for (int tile = pair_id; tile < num_tiles && ok; tile += num_pairs, ++local_tile) {
      int local;
      const GemmProblem* pr = problem_of(ps, tile, local);
      const int M = pr->M, N = pr->N;
      const float* sa = pr->sa;
      const float* sw = pr->sw;
      const __nv_bfloat16* bias = pr->bias;
      int mi, ni;
      tile_coords(local, pr->m_tiles, pr->n_tiles, pr->group_m, mi, ni);
      const int m0 = mi * P_BM + (int)rank * 128;
      const int bn = pr->bn;
      const int n0 = ni * bn;
      const uint32_t buf = local_tile & 1u;
      const uint32_t use = local_tile >> 1;
      asm volatile("bar.sync 1, %0;" ::"n"(EPI_THREADS) : "memory");
      for (int c = et; c < bn; c += EPI_THREADS) {
        const int col = n0 + c;
        s_colscale[c] = col < N ? __ldg(sw + col) : 0.f;
        s_bias[c] = (bias != nullptr && col < N) ? bias[col] : __float2bfloat16(0.f);
      }
      ok = pair_wait(&gb->acc_full[buf], use & 1u, gb, status_word, 14);
      ok = epi_all(ok);
      if (!ok) break;
      tcgen05_fence_after();

      const int row = m0 + quarter * 32 + lane;
      const float rs = row < M ? __ldg(sa + row) : 0.f;
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * BN;
      epilogue_rows(&pr->map_out, pr->out, pr->ld_out, s_staging + quarter * 2 * OUT_BLOCK_BYTES, taddr, rs,
                    s_colscale, s_bias, m0 + quarter * 32, n0, M, N, bn, pr->act_col, lane, blocks_done);
      tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&gb->acc_empty[buf]), 0));
    }
    if (lane == 0) bulk_wait_group_all();
    __syncwarp();
  }

  tcgen05_fence_before();
  __syncthreads();
  cluster_sync_all();  // neither CTA leaves while the other may still touch its shared memory or TMEM
  if (warp == 1) {
    tcgen05_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS)
                 : "memory");
  }
}

// ---- few-row product (M <= 4): weight streaming on the CUDA cores ------------------------------------
// The adaLN modulation linears see one row per image (M = batch).  A 128-row tensor-core tile would be
// 99 % padding and the tile grid (N / 256 CTAs) too small to pull the weights at HBM speed, so these
// products stream the weight matrix once with every SM: a warp owns output columns, lanes read 16-byte
// pieces of the weight row, e4m3 -> f16 (exact) -> fp32 multiply-add against the activation rows staged
// in shared memory as f16, one shuffle reduction per column.  HBM-bound: N*K bytes.
constexpr int GEMV_MAX_M = 4;
constexpr int GEMV_THREADS = 256;

__device__ __forceinline__ void e4m3x4_to_float4(uint32_t w, float (&f)[4]) {
  const __half2_raw lo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w & 0xffffu), __NV_E4M3);
  const __half2_raw hi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)(w >> 16), __NV_E4M3);
  const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&lo));
  const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&hi));
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
}

template <int TM>
__global__ void __launch_bounds__(GEMV_THREADS)
    fp8_gemv_rowscaled_kernel(const uint8_t* __restrict__ a_q, const float* __restrict__ sa,
                              const uint8_t* __restrict__ w_q, const float* __restrict__ sw,
                              const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ out, int N, int K,
                              int64_t ld_out) {
  // Activations as f16 in shared memory, laid out so that a warp's reads are conflict-free: a lane
  // needs the 16 values of "its" 16-byte weight piece = two 16-byte reads; all first halves of a row are
  // stored contiguously, then all second halves: s_a[((m * 2 + half) * chunks + chunk) * 8 + i].
  extern __shared__ __align__(16) __half s_a[];
  const int chunks = K >> 4;  // 16-byte pieces per weight row
  for (int i = threadIdx.x; i < TM * K / 4; i += GEMV_THREADS) {
    float f[4];
    e4m3x4_to_float4(reinterpret_cast<const uint32_t*>(a_q)[i], f);
    const int e = i * 4, m = e / K, k = e - m * K;  // 4 consecutive elements never straddle a half
    const int c = k >> 4, pos = k & 15;
    __half2* dst = reinterpret_cast<__half2*>(s_a + ((int64_t)(m * 2 + (pos >> 3)) * chunks + c) * 8 + (pos & 7));
    dst[0] = __floats2half2_rn(f[0], f[1]);
    dst[1] = __floats2half2_rn(f[2], f[3]);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31;
  const int warp = (blockIdx.x * GEMV_THREADS + threadIdx.x) >> 5;
  const int nwarps = (gridDim.x * GEMV_THREADS) >> 5;
  const uint4* s_a4 = reinterpret_cast<const uint4*>(s_a);
  for (int n = warp; n < N; n += nwarps) {
    const uint4* wrow = reinterpret_cast<const uint4*>(w_q + (int64_t)n * K);
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
          const uint32_t words[4] = {wv[j].x, wv[j].y, wv[j].z, wv[j].w};
          float wf[16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            float t[4];
            e4m3x4_to_float4(words[q], t);
            wf[4 * q] = t[0]; wf[4 * q + 1] = t[1]; wf[4 * q + 2] = t[2]; wf[4 * q + 3] = t[3];
          }
#pragma unroll
          for (int m = 0; m < TM; ++m) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const uint4 av = s_a4[(int64_t)(m * 2 + h) * chunks + c];
              const uint32_t aw[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 a2 = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
                acc[m] = fmaf(wf[8 * h + 2 * i], a2.x, acc[m]);
                acc[m] = fmaf(wf[8 * h + 2 * i + 1], a2.y, acc[m]);
              }
            }
          }
        }
      }
    }
#pragma unroll
    for (int m = 0; m < TM; ++m) acc[m] = warp_sum(acc[m]);
    if (lane == 0) {
      const float cs = __ldg(sw + n);
      const float b = bias != nullptr ? __bfloat162float(bias[n]) : 0.f;
#pragma unroll
      for (int m = 0; m < TM; ++m)
        out[(int64_t)m * ld_out + n] = __float2bfloat16_rn(acc[m] * __ldg(sa + m) * cs + b);
    }
  }
}

// ---- host side -----------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// Row-major 2-D tensor map with the 128-byte swizzle.  Operands: [rows, K] bytes, box = 128 bytes
// of K x box_rows, zero fill.  Output: [M, N] bf16 with a row pitch, box = 64 columns x 32 rows.
static bool make_map(CUtensorMap* map, CUtensorMapDataType type, uint32_t elem_bytes, const void* base,
                     uint64_t rows, uint64_t inner, uint64_t pitch_elems, uint32_t box_inner, uint32_t box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  cuuint64_t dims[2] = {inner, rows};
  cuuint64_t strides[1] = {pitch_elems * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, type, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS;
}

struct MapKey {
  const void* p;
  uint64_t rows, inner, pitch;
  uint32_t box_rows, elem_bytes;
  bool operator==(const MapKey& o) const {
    return p == o.p && rows == o.rows && inner == o.inner && pitch == o.pitch && box_rows == o.box_rows &&
           elem_bytes == o.elem_bytes;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.p) ^ (k.rows * 0x9E3779B97F4A7C15ull) ^ (k.inner << 20) ^ (k.pitch << 40) ^
           k.box_rows ^ ((uint64_t)k.elem_bytes << 12);
  }
};

// Encoding a tensor map costs a few microseconds of host time; weights keep their address for the
// life of the model, activations come from a caching allocator, so a small cache hits almost always.
static bool cached_map(CUtensorMap* out, const MapKey& key) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return true;
  }
  CUtensorMap m;
  const bool ok = key.elem_bytes == 1
                      ? make_map(&m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, key.p, key.rows, key.inner, key.pitch, BK,
                                 key.box_rows)
                      : make_map(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, key.p, key.rows, key.inner, key.pitch,
                                 OUT_BOX_COLS, key.box_rows);
  if (!ok) return false;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return true;
}
static bool operand_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t k, uint32_t box_rows) {
  return cached_map(out, MapKey{base, rows, k, k, box_rows, 1});
}
static bool output_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t pitch) {
  return cached_map(out, MapKey{base, rows, cols, pitch, (uint32_t)OUT_BOX_ROWS, 2});
}

static int tile_group_rows(int64_t m_tiles) {
  if (m_tiles <= 24) return (int)m_tiles;
  const int64_t groups = (m_tiles + 15) / 16;
  return (int)((m_tiles + groups - 1) / groups);
}

}  // namespace cdb

using namespace cdb;

struct cdb_gemm_problem_abi {  // mirrors `cdb_gemm_problem` of the public header
  const void* a_q;
  const float* a_scale;
  const void* w_q;
  const float* w_scale;
  const void* bias;
  void* out;
  int64_t M, N, K, ld_out;
};

static int check_problem(const cdb_gemm_problem_abi& g) {
  if (!g.a_q || !g.a_scale || !g.w_q || !g.w_scale || !g.out || g.M < 0 || g.N <= 0 || g.K <= 0 || g.ld_out < g.N)
    return CDB_ERR_BAD_ARGUMENT;
  if (g.K % 16 != 0 || g.N % 8 != 0 || g.ld_out % 8 != 0 || !aligned16(g.a_q) || !aligned16(g.w_q) ||
      !aligned16(g.out) || g.M > INT32_MAX || g.N > INT32_MAX || g.K > INT32_MAX)
    return CDB_ERR_UNSUPPORTED;
  return CDB_OK;
}

// Tuning / testing knob: a fixed tile width (0 = choose by the cost model).  Initialised from CDB_GEMM_BN.
static std::atomic<int> g_forced_tile_cols{[] {
  const char* env = getenv("CDB_GEMM_BN");
  const int v = env ? atoi(env) : 0;
  return (v >= 16 && v <= BN && v % 16 == 0) ? v : 0;
}()};

// Tuning / testing knob: 0 = choose by shape, 1 = single-CTA kernel, 2 = CTA-pair kernel.  Initialised from
// CDB_GEMM_KERNEL ("1cta" | "2cta").
static std::atomic<int> g_forced_kernel{[] {
  const char* env = getenv("CDB_GEMM_KERNEL");
  if (env && strcmp(env, "1cta") == 0) return 1;
  if (env && strcmp(env, "2cta") == 0) return 2;
  return 0;
}()};

extern "C" int cdb_tuning_set_gemm_kernel(int kind) {
  if (kind < 0 || kind > 2) return CDB_ERR_BAD_ARGUMENT;
  g_forced_kernel.store(kind, std::memory_order_relaxed);
  return CDB_OK;
}

extern "C" int cdb_tuning_set_gemm_tile_cols(int cols) {
  if (cols != 0 && (cols < 16 || cols > BN || cols % 16 != 0)) return CDB_ERR_BAD_ARGUMENT;
  g_forced_tile_cols.store(cols, std::memory_order_relaxed);
  return CDB_OK;
}

// Tile width of the single-CTA kernel for one launch.  With 128-row tiles a rank shard of a context-parallel
// run has only 3-18 row tiles, and at the full width of 256 columns the tile count often leaves most of the
// last wave idle (576 x 3072: 60 tiles on 148 SMs; 576 x 9216: 180 tiles = 1.2 waves).  A narrower tile fills
// the waves but buys less than its width suggests: timed on rank-shard shapes (cold weights, 576 - 2304 rows,
// widths 128 / 192 / 256) a K block of a tile takes about 760 + bn clocks, i.e. mostly a width-independent
// part.  So the width is the multiple of 16 that minimises
//     waves x (K blocks x (760 + 1.04 x bn) + epilogue per 64 columns) + launch,
// and the full width wins ties and anything within 3 %, so tall problems keep the shape they were tuned with.
static int choose_tile_cols(const cdb_gemm_problem_abi* g, int n, int sms, double* cost_out) {
  const int forced = g_forced_tile_cols.load(std::memory_order_relaxed);
  auto cost_of = [&](int bn) {
    int64_t tiles = 0;
    double per_tile = 0.0;
    for (int i = 0; i < n; ++i) {
      const int64_t mt = (g[i].M + BM - 1) / BM, nt = (g[i].N + bn - 1) / bn, kb = (g[i].K + BK - 1) / BK;
      tiles += mt * nt;
      const double per_kb = 760.0 + 1.04 * bn;
      const double t = kb * per_kb + 150.0 * ((bn + 63) / 64);
      per_tile = t > per_tile ? t : per_tile;
    }
    const int64_t waves = (tiles + sms - 1) / sms;
    return waves * per_tile + 3000.0;
  };
  if (forced) {
    *cost_out = cost_of(forced);
    return forced;
  }
  int best = BN;
  double best_cost = 0.97 * cost_of(BN);
  for (int bn = BN - 16; bn >= 64; bn -= 16) {
    const double c = cost_of(bn);
    if (c < best_cost) {
      best = bn;
      best_cost = c;
    }
  }
  *cost_out = best == BN ? cost_of(BN) : best_cost;
  return best;
}

// The same model for the CTA-pair kernel (256 x 256 tiles, one per pair of SMs): a K block of a pair tile takes
// about 875 clocks on the same shapes, against 1026 for a single-CTA tile of that width (a CTA of a pair takes in
// only its half of the weight tile, and the smaller stage gives its ring 6 stages instead of 4).  A pair tile
// is the cheaper one, and what decides is the wave count: 256-row tiles waste up to a tile of rows (576 rows =
// 2.25 tiles) and there are half as many tile slots.  The pair kernel also wins near-ties (within 8 %): where
// one wave is not full, the narrow single-CTA tiles the model would pick gain nothing in practice (576 x 3072 x
// 15360: 58.5 us at 112 columns as at 256, 50.8 us with pairs).
// Pair tiles may be narrower than 256 columns (a multiple of 32: each CTA holds half of the weight tile), but only
// when forced (tuning knobs): timed on the rank-shard shapes a K block of a pair tile takes 0.39 - 0.44 us at 128,
// 192 and 256 columns alike, with or without its loads, so a narrower tile never buys back what its extra tiles
// cost (576 x 3072 x 15360, 36 wide tiles for 74 pairs: 53.7 / 52.4 / 53.3 us at 256 / 192 / 128 columns;
// 2304 x 21504 x 3072: 128 / 159 / 217 us).
static double pair_cost(const cdb_gemm_problem_abi* g, int n, int sms) {
  int64_t tiles = 0;
  double per_tile = 0.0;
  for (int i = 0; i < n; ++i) {
    const int64_t mt = (g[i].M + P_BM - 1) / P_BM, nt = (g[i].N + BN - 1) / BN, kb = (g[i].K + BK - 1) / BK;
    tiles += mt * nt;
    const double t = kb * 875.0 + 150.0 * (BN / 64);
    per_tile = t > per_tile ? t : per_tile;
  }
  const int64_t slots = sms / 2 > 0 ? sms / 2 : 1;
  const int64_t waves = (tiles + slots - 1) / slots;
  return waves * per_tile + 3000.0;
}

// Which tile kernel a launch takes and at which tile width (host arithmetic only).  CTA pairs for tall problems;
// below 4096 rows (rank shards of a context-parallel run: 2304, 1152, 576 rows) whichever kernel the wave-count
// model expects to finish first.  `g` holds the problems with rows > 0, the one with more rows first.
static int plan_launch(const cdb_gemm_problem_abi* g, int n, int sms, bool* pair_out, int* bn_out) {
  const int mode = g_forced_kernel.load(std::memory_order_relaxed);
  double single_cost = 0.0;
  const int single_bn = choose_tile_cols(g, n, sms, &single_cost);
  // a forced width means the single-CTA kernel, unless the pair kernel is forced as well (then: a multiple of 32)
  const int forced_cols = g_forced_tile_cols.load(std::memory_order_relaxed);
  int pair_bn = BN;
  const double pair_c = pair_cost(g, n, sms);
  if (mode == 2 && forced_cols != 0) {
    if (forced_cols % 32 != 0) return CDB_ERR_UNSUPPORTED;
    pair_bn = forced_cols;
  }
  const bool pair = mode == 2 || (mode == 0 && CDB_GEMM_DEFAULT_PAIR &&
                                  (g[0].M >= 4096 || (forced_cols == 0 && pair_c < 1.08 * single_cost)));
  *pair_out = pair;
  *bn_out = pair ? pair_bn : single_bn;
  return CDB_OK;
}

// The plan of a launch without launching it: kind 1 = single-CTA tile kernel, 2 = CTA-pair kernel, 3 = few-row
// weight-streaming kernel.  Touches no GPU: `sm_count` is given (148 on a B200).
extern "C" int cdb_fp8_gemm_plan(const void* problems_v, int count, int sm_count_hint, int* kind, int* tile_cols) {
  const cdb_gemm_problem_abi* in = static_cast<const cdb_gemm_problem_abi*>(problems_v);
  if (!in || !kind || !tile_cols || count < 1 || count > MAX_PROBLEMS || sm_count_hint < 2) return CDB_ERR_BAD_ARGUMENT;
  cdb_gemm_problem_abi g[MAX_PROBLEMS];
  int n = 0;
  for (int i = 0; i < count; ++i) {
    if (in[i].M < 0 || in[i].N <= 0 || in[i].K <= 0) return CDB_ERR_BAD_ARGUMENT;
    if (in[i].M > 0) g[n++] = in[i];
  }
  *kind = 0;
  *tile_cols = 0;
  if (n == 0) return CDB_OK;
  if (n == 2 && g[1].M > g[0].M) std::swap(g[0], g[1]);
  if (n == 1 && g_forced_kernel.load(std::memory_order_relaxed) == 0 && g[0].M <= GEMV_MAX_M &&
      g[0].M * g[0].K * 2 <= 48 * 1024) {
    *kind = 3;
    return CDB_OK;
  }
  bool pair = false;
  const int rc = plan_launch(g, n, sm_count_hint, &pair, tile_cols);
  *kind = pair ? 2 : 1;
  return rc;
}

static int launch_few_rows(const cdb_gemm_problem_abi& g, int sms, cudaStream_t st) {
  const uint8_t* ap = static_cast<const uint8_t*>(g.a_q);
  const uint8_t* wp = static_cast<const uint8_t*>(g.w_q);
  const __nv_bfloat16* bp = static_cast<const __nv_bfloat16*>(g.bias);
  __nv_bfloat16* op = static_cast<__nv_bfloat16*>(g.out);
  const int64_t want = (g.N + GEMV_THREADS / 32 - 1) / (GEMV_THREADS / 32);
  const unsigned grid = (unsigned)(want < (int64_t)sms * 4 ? want : (int64_t)sms * 4);
  const size_t smem = (size_t)g.M * g.K * 2;
#define CDB_GEMV(TM)                                                                                          \
  fp8_gemv_rowscaled_kernel<TM><<<grid, GEMV_THREADS, smem, st>>>(ap, g.a_scale, wp, g.w_scale, bp, op, (int)g.N, \
                                                                  (int)g.K, g.ld_out)
  if (g.M == 1) CDB_GEMV(1);
  else if (g.M == 2) CDB_GEMV(2);
  else if (g.M == 3) CDB_GEMV(3);
  else CDB_GEMV(4);
#undef CDB_GEMV
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

// Up to two products in one launch of the tile kernels; the one with more rows goes first.  `gelu_from_col`
// (may be null) gives, per problem, the first output column that passes through tanh-GELU in the epilogue.
extern "C" int cdb_fp8_gemm_rowscaled_grouped_act(const void* problems_v, int count, const int64_t* gelu_from_col,
                                                  int32_t* status_word, void* stream) {
  const cdb_gemm_problem_abi* in = static_cast<const cdb_gemm_problem_abi*>(problems_v);
  if (!in || count < 1 || count > MAX_PROBLEMS) return CDB_ERR_BAD_ARGUMENT;
  cdb_gemm_problem_abi g[MAX_PROBLEMS];
  int act[MAX_PROBLEMS];
  int n = 0;
  bool any_act = false;
  for (int i = 0; i < count; ++i) {
    const int rc = check_problem(in[i]);
    if (rc != CDB_OK) return rc;
    int a = INT32_MAX;
    if (gelu_from_col != nullptr && gelu_from_col[i] >= 0 && gelu_from_col[i] < in[i].N) {
      if (gelu_from_col[i] % 8 != 0) return CDB_ERR_UNSUPPORTED;  // the epilogue decides per 16-byte chunk
      a = (int)gelu_from_col[i];
    }
    if (in[i].M > 0) {
      any_act = any_act || a != INT32_MAX;
      act[n] = a;
      g[n++] = in[i];
    }
  }
  if (n == 0) return CDB_OK;
  if (n == 2 && g[1].M > g[0].M) {
    std::swap(g[0], g[1]);
    std::swap(act[0], act[1]);
  }
  // The opt-in to more than 48 KB of dynamic shared memory is a per-device function attribute.
  static PerDevice attr_state;
  const cudaError_t attr_err = (cudaError_t)attr_state.get([]() -> int64_t {
    cudaError_t e = cudaFuncSetAttribute(fp8_gemm_rowscaled_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_TOTAL_BYTES);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(fp8_gemm_rowscaled_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               P_SMEM_TOTAL_BYTES);
    return (int64_t)e;
  });
  const int mode = g_forced_kernel.load(std::memory_order_relaxed);
  CDB_CUDA_CHECK(attr_err);
  const int sms = sm_count();
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (n == 1 && mode == 0 && !any_act && g[0].M <= GEMV_MAX_M && g[0].M * g[0].K * 2 <= 48 * 1024)
    return launch_few_rows(g[0], sms, st);
  bool pair = false;
  int bn = BN;
  const int plan_rc = plan_launch(g, n, sms, &pair, &bn);
  if (plan_rc != CDB_OK) return plan_rc;
  const int64_t tile_rows = pair ? P_BM : BM;
  GemmProblems ps{};
  ps.count = n;
  int64_t tiles = 0;
  for (int i = 0; i < n; ++i) {
    GemmProblem& o = ps.p[i];
    const uint32_t a_box = pair ? 128 : BM, w_box = pair ? (uint32_t)bn / 2 : (uint32_t)bn;
    if (!operand_map(&o.map_a, g[i].a_q, (uint64_t)g[i].M, (uint64_t)g[i].K, a_box) ||
        !operand_map(&o.map_w, g[i].w_q, (uint64_t)g[i].N, (uint64_t)g[i].K, w_box) ||
        !output_map(&o.map_out, g[i].out, (uint64_t)g[i].M, (uint64_t)g[i].N, (uint64_t)g[i].ld_out)) {
      set_cuda_error(cudaErrorUnknown, "cuTensorMapEncodeTiled");
      return CDB_ERR_CUDA;
    }
    o.sa = g[i].a_scale;
    o.sw = g[i].w_scale;
    o.bias = static_cast<const __nv_bfloat16*>(g[i].bias);
    o.M = (int)g[i].M;
    o.N = (int)g[i].N;
    o.K = (int)g[i].K;
    o.m_tiles = (int)((g[i].M + tile_rows - 1) / tile_rows);
    o.out = static_cast<__nv_bfloat16*>(g[i].out);
    o.ld_out = g[i].ld_out;
    o.bn = bn;
    o.idesc = pair ? idesc_e4m3_f32(P_BM, bn) : idesc_e4m3_f32(BM, bn);
    o.n_tiles = (int)((g[i].N + bn - 1) / bn);
    o.k_blocks = (int)((g[i].K + BK - 1) / BK);
    o.group_m = tile_group_rows(o.m_tiles);
    o.tile_begin = (int)tiles;
    o.act_col = act[i];
    tiles += (int64_t)o.m_tiles * o.n_tiles;
  }
  if (tiles > INT32_MAX) return CDB_ERR_TOO_LARGE;
  ps.num_tiles = (int)tiles;
  ps.stage_bytes = A_STAGE_BYTES + bn * BK;
  ps.stages = SMEM_TILE_BYTES / ps.stage_bytes < MAX_STAGES ? SMEM_TILE_BYTES / ps.stage_bytes : MAX_STAGES;
  if (pair) {
    const int64_t pairs = tiles < sms / 2 ? tiles : sms / 2;
    fp8_gemm_rowscaled_pair_kernel<<<(unsigned)(2 * pairs), GEMM_THREADS, P_SMEM_TOTAL_BYTES, st>>>(ps, status_word);
  } else {
    const unsigned grid = (unsigned)(tiles < sms ? tiles : sms);
    fp8_gemm_rowscaled_kernel<<<grid, GEMM_THREADS, SMEM_TOTAL_BYTES, st>>>(ps, status_word);
  }
  CDB_CUDA_CHECK(cudaGetLastError());
  return CDB_OK;
}

extern "C" int cdb_fp8_gemm_rowscaled_grouped(const void* problems_v, int count, int32_t* status_word, void* stream) {
  return cdb_fp8_gemm_rowscaled_grouped_act(problems_v, count, nullptr, status_word, stream);
}

extern "C" int cdb_fp8_gemm_rowscaled(const void* a_q, const float* a_scale, const void* w_q,
                                      const float* w_scale, const void* bias, void* out, int64_t M,
                                      int64_t N, int64_t K, int64_t ld_out, int32_t* status_word,
                                      void* stream) {
  const cdb_gemm_problem_abi g{a_q, a_scale, w_q, w_scale, bias, out, M, N, K, ld_out};
  return cdb_fp8_gemm_rowscaled_grouped_act(&g, 1, nullptr, status_word, stream);
}
