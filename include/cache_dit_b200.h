/*
 * C ABI of the B200 (sm_100a) hot-path kernels behind cache-dit's public Python API.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream handle
 * (a cudaStream_t passed as void*), enqueues work on that stream and returns a
 * status code (0 = success).  Nothing here allocates device memory unless stated;
 * the caller owns all buffers.  There is no CPU fallback: the functions need a
 * CUDA device of compute capability 10.0.
 *
 * Each declaration names the part of the reference (vipshop/cache-dit, paths
 * inside that project) whose eager PyTorch code it replaces.
 */
#ifndef CACHE_DIT_B200_H_
#define CACHE_DIT_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define CDB_API __attribute__((visibility("default")))
#else
#define CDB_API
#endif

/* Storage dtype of activation tensors. */
enum cdb_dtype { CDB_F32 = 0, CDB_BF16 = 1, CDB_F16 = 2 };

/* Status codes. */
enum cdb_status {
  CDB_OK = 0,
  CDB_ERR_BAD_ARGUMENT = 1,   /* null pointer, negative size, unknown dtype, ... */
  CDB_ERR_UNSUPPORTED = 2,    /* shape or alignment the kernel does not cover */
  CDB_ERR_SCRATCH_TOO_SMALL = 3,
  CDB_ERR_CUDA = 4,           /* a CUDA runtime / driver call failed; see cdb_last_cuda_error */
  CDB_ERR_NO_DEVICE = 5,      /* no sm_100 device is current */
  CDB_ERR_DEVICE_TIMEOUT = 6, /* a bounded device-side wait ran out (read from a status word) */
  CDB_ERR_TOO_LARGE = 7       /* a size beyond the stated maximum of the entry point */
};

#define CDB_MAX_TAYLOR_TERMS 5 /* Taylor order <= 4: terms dY[0..4] */

CDB_API int cdb_abi_version(void);
CDB_API const char* cdb_status_string(int status);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
CDB_API const char* cdb_last_cuda_error(void);

/* ------------------------------------------------------------------------------------------
 * Relative-L1 check.  Replaces
 *   Fn residual formation           src/cache_dit/caching/cache_blocks/pattern_base.py:195
 *   (t1-t2).abs().mean(), t1.abs().mean()
 *                                   src/cache_dit/caching/cache_contexts/cache_manager.py:609-610
 * One pass over the tensors:
 *   r      = base ? round_dtype(cur - base) : cur          (n elements of `dtype`)
 *   if residual_out: residual_out = r
 *   if prev:  means[0] = round_dtype( sum |round_dtype(prev - r)| / n )
 *             means[1] = round_dtype( sum |prev| / n )
 * `means` is two float32 on the device.  They are the two 0-dim tensors the reference
 * all-reduces (cache_manager.py:612-614) and then divides (cache_manager.py:619).
 * `scratch` is device memory of at least cdb_rel_l1_scratch_bytes() bytes, 128-byte aligned, that
 * must be zero-filled once before its first use; the kernel leaves it zeroed for the next launch.
 * Launches that share one scratch buffer must be ordered on one stream.  One CTA of the launch collects
 * the other clusters' partial sums from the scratch with a bounded wait (2 s); should that wait ever
 * run out, both means are NaN.
 * ---------------------------------------------------------------------------------------- */
CDB_API size_t cdb_rel_l1_scratch_bytes(void);
CDB_API int cdb_rel_l1(const void* cur, const void* base, const void* prev, void* residual_out,
               int64_t n, int dtype, float* means, void* scratch, size_t scratch_bytes,
               void* stream);

/* ------------------------------------------------------------------------------------------
 * Relative-L1 check without any allocation.  No counterpart in the reference: it exists for
 * hosts that must not allocate device memory around the check (a plug-in living inside another
 * framework's memory pool, a process whose device memory is pre-partitioned, a serving loop with
 * a no-allocation-after-warm-up rule) and therefore cannot supply cdb_rel_l1's scratch buffer.
 *
 * Same arithmetic and outputs as cdb_rel_l1 with `prev` given (means[0], means[1], optional
 * residual_out); the reduction scratch is a fixed array inside the library's device image
 * (cdb_rel_l1_scratch_bytes() = 16384 bytes per GPU that loads the library, held until the process exits).
 *   - The device that owns the tensors must be the current device of the calling thread: the array
 *     exists once per device and the current device's copy is used.  A `cur` that is not device memory
 *     of the current device returns CDB_ERR_BAD_ARGUMENT.
 *   - n may not exceed CDB_REL_L1_STATIC_MAX_ELEMS; larger calls return CDB_ERR_TOO_LARGE and the
 *     reason is available from cdb_last_cuda_error().
 *   - The first call on each device looks up the array's device address (with that device
 *     current).  Make that first call outside of any CUDA stream capture.
 *   - All calls on a device share the one array.  Calls must not overlap on the GPU: issue them
 *     on one stream, or order the streams yourself; overlapping launches race on the scratch and
 *     give wrong means.
 *   - The entry point calls no cudaMalloc / cudaFree and no library routine that allocates.
 * ---------------------------------------------------------------------------------------- */
#define CDB_REL_L1_STATIC_MAX_ELEMS ((int64_t)1 << 30)
CDB_API int cdb_rel_l1_static(const void* cur, const void* base, const void* prev, void* residual_out,
                              int64_t n, int dtype, float* means, void* stream);

/* ------------------------------------------------------------------------------------------
 * Cached-residual apply.  Replaces
 *   TaylorSeerState.approximate     src/cache_dit/caching/cache_contexts/calibrators/taylorseer.py:91-104
 *   hidden_states_prev + hidden_states
 *                                   src/cache_dit/caching/cache_contexts/cache_manager.py:830-834
 *   approx = sum_i round(round(coef[i] * derivs[i]) * power[i])      (rounded after every op)
 *   out    = add_hidden ? round(approx + hidden) : approx
 * coef[i] = 1/i!, power[i] = elapsed^i are supplied by the host.  `out` may alias `hidden`.
 * n_terms in [1, CDB_MAX_TAYLOR_TERMS]; a plain (non-Taylor) cached buffer is n_terms = 1.
 * ---------------------------------------------------------------------------------------- */
CDB_API int cdb_taylor_apply(const void* hidden, const void* const* derivs, const float* coef,
                     const float* power, int n_terms, int add_hidden, void* out, int64_t n,
                     int dtype, void* stream);

/* ------------------------------------------------------------------------------------------
 * TaylorSeer derivative update.  Replaces
 *   Mn residual formation           src/cache_dit/caching/cache_blocks/pattern_base.py:414,418
 *   TaylorSeerState.derivative      src/cache_dit/caching/cache_contexts/calibrators/taylorseer.py:68-89
 *   y       = before ? round(after - before) : after
 *   cur[0]  = y                      (written unless cur[0] == after and before == NULL)
 *   cur[i+1]= round(round(cur[i] - prev[i]) / window)   for i < n_new
 * n_new in [0, CDB_MAX_TAYLOR_TERMS-1]: how many finite differences the host state allows.
 * `cur[*]` must not alias `prev[*]`.
 * ---------------------------------------------------------------------------------------- */
CDB_API int cdb_taylor_update(const void* after, const void* before, const void* const* prev,
                      void* const* cur, int n_new, float window, int64_t n, int dtype,
                      void* stream);

/* ------------------------------------------------------------------------------------------
 * Per-row dynamic FP8 (e4m3fn) quantization.  Replaces torchao's dynamic activation
 * quantization selected by the reference at
 *   src/cache_dit/quantization/torchao/quantize_ao.py:540-558  (PerRow, e4m3, zero scale -> 1 at :43-71)
 *   scale[r] = amax_r * fl32(1/448) (PyTorch's CUDA `amax / 448.0`; 1 if the row is all zero);
 *   q = saturate_e4m3(x / scale[r])
 * x is [rows, cols] bf16 row-major with row stride `ld_x` elements; q is [rows, cols] bytes,
 * contiguous; scale is [rows] float32.  Also used once per weight at load time ([N, K] rows).
 * ---------------------------------------------------------------------------------------- */
CDB_API int cdb_fp8_quant_rows(const void* x, int64_t rows, int64_t cols, int64_t ld_x, void* q,
                       float* scale, void* stream);

/* Producer-fused variants: the bf16 tensor the reference would write and re-read is never
 * materialised.  pre-op selects what is applied to each element before quantization.
 *   CDB_PRE_LAYERNORM_MOD: y = layernorm(x_row, eps) * (1 + mod_scale[b]) + mod_shift[b]
 *                          (adaLN-modulated LayerNorm without affine; b = row / rows_per_batch)
 *   CDB_PRE_GELU_TANH:     y = gelu_tanh(x)
 * Intermediate y is rounded to bf16 before quantization, as the unfused bf16 pipeline does. */
enum cdb_preop {
  CDB_PRE_NONE = 0,
  CDB_PRE_LAYERNORM_MOD = 1,
  CDB_PRE_GELU_TANH = 2,
  CDB_PRE_CONCAT_GELU = 3 /* internal to cdb_fp8_quant_rows_concat_gelu; rejected by ..._fused */
};
CDB_API int cdb_fp8_quant_rows_fused(const void* x, int64_t rows, int64_t cols, int64_t ld_x, int preop,
                             const void* mod_shift, const void* mod_scale, int64_t rows_per_batch,
                             int64_t ld_mod, float eps, void* q, float* scale, void* stream);

/* Up to two independent products in one launch: the tiles of the one with fewer rows come last and fill
 * the SMs that the other's final, partial wave leaves idle (the text stream of a double-stream block beside
 * the image stream's product of the same layer).  Same arithmetic and requirements per problem as
 * cdb_fp8_gemm_rowscaled. */
typedef struct cdb_gemm_problem {
  const void* a_q;
  const float* a_scale;
  const void* w_q;
  const float* w_scale;
  const void* bias;
  void* out;
  int64_t M, N, K, ld_out;
} cdb_gemm_problem;
CDB_API int cdb_fp8_gemm_rowscaled_grouped(const void* problems /* cdb_gemm_problem[count] */, int count,
                                   int32_t* status_word, void* stream);
/* The same launch with an activation in the epilogue (no counterpart in the reference, where the MLP's GELU is
 * an eager op of the wrapped block): for problem i, output columns >= gelu_from_col[i] are written as
 * bf16(gelu_tanh(bf16(product))), i.e. what `gelu(linear(x))` gives in bf16, so the tensor a following
 * quantization reads needs no activation pass of its own.  gelu_from_col may be NULL; an entry that is negative
 * or >= N means no activation for that problem; other entries must be multiples of 8.  0 activates the whole
 * output (an MLP-in projection), the offset of a member activates one member of a concatenated product (the
 * MLP-in columns behind q/k/v). */
CDB_API int cdb_fp8_gemm_rowscaled_grouped_act(const void* problems /* cdb_gemm_problem[count] */, int count,
                                       const int64_t* gelu_from_col, int32_t* status_word, void* stream);

/* cdb_fp8_quant_rows_fused on two tensors of the same width in one launch (image and text stream of a
 * double-stream block): each has its own rows, row stride, modulation vectors (LayerNorm variant) and
 * outputs.  preop is CDB_PRE_NONE, CDB_PRE_LAYERNORM_MOD or CDB_PRE_GELU_TANH. */
CDB_API int cdb_fp8_quant_rows_fused_pair(const void* x, int64_t rows, int64_t ld_x, const void* mod_shift,
                                  const void* mod_scale, int64_t rows_per_batch, int64_t ld_mod, void* q,
                                  float* scale, const void* x2, int64_t rows2, int64_t ld_x2,
                                  const void* mod_shift2, const void* mod_scale2, int64_t rows_per_batch2,
                                  int64_t ld_mod2, void* q2, float* scale2, int64_t cols, int preop, float eps,
                                  void* stream);

/* Quantizes the rows of the concatenation [head | gelu_tanh(tail)] without building it: the input
 * of a parallel attention + MLP block's output projection (attention output beside the activated
 * MLP branch).  head [rows, head_cols] and tail [rows, tail_cols] are bf16 with their own row
 * strides; q is [rows, head_cols + tail_cols] contiguous; one scale per whole row.
 * Column counts and strides must be multiples of 8; at most 24576 columns in total. */
CDB_API int cdb_fp8_quant_rows_concat_gelu(const void* head, int64_t head_cols, int64_t ld_head,
                                   const void* tail, int64_t tail_cols, int64_t ld_tail,
                                   int64_t rows, void* q, float* scale, void* stream);
/* The same for [head | tail] with a tail that already is activated (written by
 * cdb_fp8_gemm_rowscaled_grouped_act): concatenation and quantization only. */
CDB_API int cdb_fp8_quant_rows_concat(const void* head, int64_t head_cols, int64_t ld_head, const void* tail,
                              int64_t tail_cols, int64_t ld_tail, int64_t rows, void* q, float* scale,
                              void* stream);

/* ------------------------------------------------------------------------------------------
 * Row-scaled FP8 GEMM.  Replaces the torch._scaled_mm call at
 *   src/cache_dit/quantization/torchao/_scaled_mm.py:62-91
 *   out[m, n] = (sum_k a_q[m, k] * w_q[n, k]) * a_scale[m] * w_scale[n] (+ bias[n])
 * a_q [M, K] e4m3 row-major, w_q [N, K] e4m3 row-major (the linear layer's weight layout),
 * scales float32, bias bf16 or NULL, out [M, N] bf16 row-major with row stride ld_out.
 * Requirements: K % 16 == 0, N % 8 == 0, pointers 16-byte aligned.  Accumulation is fp32 in
 * tensor memory (tcgen05).  `status_word` (device int32, may be NULL) receives a non-zero
 * value if a bounded in-kernel wait expired.
 * ---------------------------------------------------------------------------------------- */
CDB_API int cdb_fp8_gemm_rowscaled(const void* a_q, const float* a_scale, const void* w_q,
                           const float* w_scale, const void* bias, void* out, int64_t M,
                           int64_t N, int64_t K, int64_t ld_out, int32_t* status_word,
                           void* stream);

/* Tuning knob (no counterpart in the reference): the single-CTA tile kernel picks its tile width,
 * a multiple of 16 columns up to 256, from a cost model so that the tiles fill whole waves of SMs; a non-zero
 * `cols` fixes the width for every later launch of the process, 0 restores the model.  The environment variable
 * CDB_GEMM_BN sets the initial value.  Results do not depend on the width (bitwise).  Together with
 * cdb_tuning_set_gemm_kernel(2) a multiple of 32 fixes the width of the CTA-pair kernel's tiles instead. */
/* What a launch of cdb_fp8_gemm_rowscaled_grouped would run for these problems on a GPU with `sm_count` SMs, without
 * launching anything or touching a GPU (only M, N, K of the problems are read): *kind = 1 single-CTA tile kernel,
 * 2 CTA-pair kernel, 3 few-row weight-streaming kernel, 0 nothing to do; *tile_cols = the tile width (0 for kind 3). */
CDB_API int cdb_fp8_gemm_plan(const void* problems /* cdb_gemm_problem[count] */, int count, int sm_count, int* kind,
                      int* tile_cols);
CDB_API int cdb_tuning_set_gemm_tile_cols(int cols);
/* Tuning knob (no counterpart in the reference): which tile kernel the FP8 product launches.  0 = chosen per
 * launch by a wave-count model, 1 = the single-CTA kernel, 2 = the CTA-pair kernel (cta_group::2).  The
 * environment variable CDB_GEMM_KERNEL ("1cta" | "2cta") sets the initial value.  Results do not depend on the
 * choice (bitwise). */
CDB_API int cdb_tuning_set_gemm_kernel(int kind);
/* ------------------------------------------------------------------------------------------
 * Transformer-block glue between the FP8 linears.  No counterpart in the reference: there these
 * are eager PyTorch ops inside the diffusers transformer blocks that cache-dit wraps.  They are
 * here because, once the linears run in FP8, these elementwise passes dominate a computed step.
 *
 * cdb_qk_norm_rope: per-head RMSNorm (weight [head_dim]) of a projected q or k, then the rotary
 * embedding, written straight into a joint [batch, total_tokens, heads, head_dim] buffer.
 *   x    [tokens, heads*head_dim] bf16, row stride ld_x (may be a column slice of a wider GEMM output)
 *   cos/sin tables [total_tokens, head_dim] bf16; row used = pos_offset + (token index in its batch)
 *   out  row (b, pos) starts at out + b*out_batch_stride + pos*ld_out
 *   y = bf16(x * rsqrt(mean(x^2) + eps) * w);  out = bf16(bf16(y*cos) + bf16(rot(y)*sin)),
 *   rot of each pair (y0, y1) = (-y1, y0).   head_dim in {64, 128, 256}; strides % 8 == 0.
 *
 * cdb_gated_residual: out[r, :] = x[r, :] + gate[r / rows_per_batch, :] * y[r, :]   (bf16, the
 * product rounded before the add).  x and out contiguous [rows, cols]; y row stride ld_y.
 * ---------------------------------------------------------------------------------------- */
CDB_API int cdb_qk_norm_rope(const void* x, int64_t ld_x, const void* norm_weight, const void* cos_table,
                     const void* sin_table, void* out, int64_t ld_out, int64_t out_batch_stride,
                     int64_t tokens, int64_t tokens_per_batch, int pos_offset, int heads,
                     int head_dim, float eps, void* stream);
CDB_API int cdb_gated_residual(const void* x, const void* y, int64_t ld_y, const void* gate,
                       int64_t ld_gate, void* out, int64_t rows, int64_t rows_per_batch,
                       int64_t cols, void* stream);

/* ------------------------------------------------------------------------------------------
 * Ulysses exchange around attention as stores into peer GPUs' memory (NVLink), fused with the
 * producer.  Replaces the four all-to-all collectives per block that the reference's context-
 * parallel plan issues through diffusers' hooks (src/cache_dit/distributed/transformers/flux.py:49-61,
 * src/cache_dit/distributed/core/_distributed_primitives.py all-to-all helpers).
 * `dst_ptrs[r]` / `flag_ptrs[r]` are addresses valid on THIS device for rank r's buffer (the own
 * buffer for r = own rank, CUDA-IPC mappings for the others); at most 8 ranks.
 *
 * cdb_scatter_heads: x [tokens, heads*head_dim] bf16 (row stride ld_x) holds this rank's tokens for
 *   all heads.  Head h is written to rank h / (heads/world) as local head h % (heads/world), joint row
 *   dst_row_offset + (token index in its batch), in a [batch, rows, heads/world, head_dim] buffer with
 *   batch stride dst_batch_stride.  With norm_weight != NULL the per-head RMSNorm + rotary embedding of
 *   cdb_qk_norm_rope is applied first (table row = table_row_offset + token index); with NULL it copies.
 *   norm_across_heads != 0: the RMS statistic is taken over the whole row and norm_weight is
 *   [heads*head_dim] (Wan's q / k normalisation) instead of per head with weight [head_dim].
 * cdb_gather_tokens: o [batch, tokens_all, heads_per_rank, head_dim] (this rank's heads, all tokens):
 *   token s goes to the rank r with row_starts[r] <= s < row_starts[r+1] (host array of world+1 entries;
 *   NULL = equal ranges), into its [batch, dst_token_capacity, heads_per_rank*world, head_dim] buffer
 *   at token s - row_starts[r] and head offset my_rank*heads_per_rank.  Ranges may differ in length.
 * cdb_peer_signal / cdb_peer_wait: `sync` is cdb_peer_sync_bytes() of zeroed device memory per rank;
 *   each rank owns `world` zeroed 32-bit flag words.  signal bumps the rank's epoch and stores it into
 *   word my_rank of every rank's flags; wait returns when all words of the own flags reached the own
 *   epoch, or after timeout_ns, in which case a status is latched in `sync` (second int32: 1 + late
 *   peer) and every later wait returns at once.  Both are single launches and may be graph-captured.
 * cdb_peer_enable_access: cudaDeviceEnablePeerAccess from the current device, idempotent.
 * ---------------------------------------------------------------------------------------- */
CDB_API int cdb_peer_enable_access(int peer_device);
/* Buffers peers can map: cudaMalloc'd and zero-filled (alloc), exported as a 64-byte CUDA IPC handle,
 * imported in another process on the same node (the returned address is valid on the importer's
 * current device; peer access is enabled by the import), released before the owner frees. */
CDB_API int cdb_peer_alloc(size_t bytes, void** out);
CDB_API int cdb_peer_free(void* p);
CDB_API int cdb_peer_export(const void* p, unsigned char* handle64);
CDB_API int cdb_peer_import(const unsigned char* handle64, void** out);
CDB_API int cdb_peer_release(void* imported);
CDB_API int cdb_scatter_heads(const void* x, int64_t ld_x, const void* norm_weight, int norm_across_heads,
                      const void* cos_table, const void* sin_table, int table_row_offset,
                      void* const* dst_ptrs, int world,
                      int64_t dst_batch_stride, int64_t tokens, int64_t tokens_per_batch,
                      int64_t dst_row_offset, int heads, int head_dim, float eps, void* stream);
/* Up to 6 cdb_scatter_heads jobs in one launch (q, k, v of the text and image stream of a block). */
typedef struct cdb_scatter_job {
  const void* x;
  int64_t ld_x, tokens, tokens_per_batch;
  const void* norm_weight; /* NULL: copy */
  int norm_across_heads;
  float eps;
  const void* cos_table;
  const void* sin_table;
  int table_row_offset;
  void* const* dst_ptrs; /* `world` addresses */
  int64_t dst_batch_stride, dst_row_offset;
  /* FP8 on the wire (the reference's `ulysses_float8`): NULL = bf16.  Otherwise dst_ptrs receive e4m3 bytes
   * in the same [batch, rows, heads/world, head_dim] layout and these `world` buffers one float32 scale per
   * (token, head): s = max(amax/448, 1e-6), q = e4m3(clamp(x / s))
   * (src/cache_dit/kernels/triton/_float8_comm.py:78-124). */
  void* const* dst_scale_ptrs;
} cdb_scatter_job;
CDB_API int cdb_scatter_heads_multi(const void* jobs /* cdb_scatter_job[njobs] */, int njobs, int world, int heads,
                            int head_dim, void* stream);
CDB_API int cdb_gather_tokens(const void* o, void* const* dst_ptrs, int world, int my_rank, int64_t batch,
                      int64_t tokens_all, const int64_t* row_starts, int64_t dst_token_capacity,
                      int heads_per_rank, int head_dim, void* stream);
/* FP8 variant of cdb_gather_tokens (per (token, head): s = max(amax, 1e-4)/448, q = e4m3(clamp(x * (1/s))),
 * scale stored as bf16; src/cache_dit/kernels/triton/_float8_comm.py:6-44 as called at
 * src/cache_dit/kernels/triton/_ops_registery.py:50-76), and the unpacking of either format on the receiver:
 * out = bf16(float(q) * scale) for up to 3 tensors of `rows[i]` rows of head_dim bytes. */
CDB_API int cdb_gather_tokens_fp8(const void* o, void* const* dst_ptrs, void* const* dst_scale_ptrs, int world,
                          int my_rank, int64_t batch, int64_t tokens_all, const int64_t* row_starts,
                          int64_t dst_token_capacity, int heads_per_rank, int head_dim, void* stream);
CDB_API int cdb_fp8_dequant_heads(const void* const* q, const void* const* scales, void* const* out,
                          const int64_t* rows, int njobs, int head_dim, int scales_are_bf16, void* stream);
CDB_API size_t cdb_peer_sync_bytes(void);
CDB_API int cdb_peer_signal(void* const* flag_ptrs, int world, int my_rank, void* sync, void* stream);
CDB_API int cdb_peer_wait(const void* my_flags, int world, void* sync, uint64_t timeout_ns, void* stream);
/* signal followed by wait as one launch */
CDB_API int cdb_peer_barrier(void* const* flag_ptrs, const void* my_flags, int world, int my_rank, void* sync,
                     uint64_t timeout_ns, void* stream);

/* Few-row bf16 product for adaLN modulation projections that stay in bf16 (the reference's name filter keeps
 * layers named *mod* out of FP8, src/cache_dit/quantization/config.py:356-361, so there they are cuBLAS calls
 * inside the diffusers block): out[m, n] = bf16(sum_k x[m, k] * w[n, k] + bias[n]) for M <= 4 rows, fp32
 * accumulation, w [N, K] bf16 row-major and 16-byte aligned, K % 8 == 0, M * K * 4 <= 48 KB.  Streams the weights
 * once; a column's result does not depend on which row slice of `w` a call covers, so a context-parallel run can
 * shard the columns over the ranks without changing a bit. */
CDB_API int cdb_bf16_gemv(const void* x, int64_t ld_x, const void* w, const void* bias, void* out, int64_t ld_out,
                          int64_t M, int64_t N, int64_t K, void* stream);

/* cdb_gated_residual on two (x, y, gate, out) sets of the same width in one launch. */
CDB_API int cdb_gated_residual_pair(const void* x, const void* y, int64_t ld_y, const void* gate, int64_t ld_gate,
                            void* out, int64_t rows, int64_t rows_per_batch, const void* x2, const void* y2,
                            int64_t ld_y2, const void* gate2, int64_t ld_gate2, void* out2, int64_t rows2,
                            int64_t rows_per_batch2, int64_t cols, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CACHE_DIT_B200_H_ */
