/* C ABI of the B200 (sm_100a) W8A8 linear path.
 *
 * Every entry point takes plain pointers and sizes.  Unless stated otherwise pointers are
 * DEVICE pointers owned by the caller, work is enqueued asynchronously on `stream`
 * (a cudaStream_t passed as void*; NULL = the legacy default stream, B200_STREAM_PER_THREAD
 * = the per-thread default stream the reference is compiled for), and the return value
 * follows the reference's operator convention (src/world_cuda_ops.cu:28-42): 0 = success,
 * 1 = failure with a message on stderr (also kept for b200_w8a8_last_error).  Nothing here
 * throws, aborts, or falls back to a CPU path.
 *
 * Each declaration names the reference interface it stands in for, as
 * path-in-reference:line.
 */
#ifndef B200_W8A8_H
#define B200_W8A8_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200_W8A8_ABI_VERSION 1

/* element types of activations / outputs */
#define B200_DT_F32 0
#define B200_DT_F16 1
#define B200_DT_BF16 2
#define B200_DT_S32 3

/* epilogue activations */
#define B200_ACT_NONE 0
#define B200_ACT_SILU 1
#define B200_ACT_GELU_TANH 2

/* int8 weight layouts.  ROW_MAJOR is the reference's int8[N,K] (src/world_cuda.cu:153-222).
 * SLAB128 stores, for each 128-byte slab of K, all N rows contiguously: [K/128][N][128];
 * a GEMM tile of any height is then one contiguous block of HBM.  Needs K % 128 == 0. */
#define B200_W_ROW_MAJOR 0
#define B200_W_SLAB128 1

#define B200_STREAM_PER_THREAD ((void *)0x2)

int b200_w8a8_abi_version(void);
/* Last failure message of the calling thread ("" if none). */
const char *b200_w8a8_last_error(void);
/* Every device-side wait of the GEMM kernels has a time limit (2 s).  A kernel whose wait runs out
 * drains, exits and leaves a code in a status word kept in pinned host memory that the device writes
 * directly; the next call of any launching entry point (the wm_cuda_* operators included) sees it with
 * a plain host load, prints the reason, returns 1 once and starts clean (it synchronizes the device,
 * clears the word and re-zeroes the ticket counters of the built-in split-K scratch; a split-K
 * workspace owned by the caller must be zeroed again by the caller).  That is the reference's
 * "non-zero on any failure" convention (src/world_cuda_ops.cu:28-42, 2856-2863) extended to
 * failures a kernel discovers after its launch returned.
 * b200_w8a8_poll_status synchronizes the current device and reports and clears the word
 * (0 = healthy; codes: KernelStatus in csrc/common.cuh). */
int b200_w8a8_poll_status(int *status_out);
/* Test aids for the failure path (no counterpart in the reference).  set_wait_limit_ns changes the
 * limit of every later launch (0 restores 2 s).  drop_operand_load makes the TMA producer of the next
 * `launches` GEMM launches leave out its first activation tile, so that the MMA issuer's wait runs
 * out and the abort path executes; nothing faults, the kernel returns with status 102. */
void b200_w8a8_debug_set_wait_limit_ns(unsigned long long ns);
void b200_w8a8_debug_drop_operand_load(int launches);

/* Self-test: the rate at which this device retires tcgen05.mma kind::i8 (128 x 256 x 32 per
 * instruction) when one CTA per SM issues `slabs_per_cta` x 4 of them back to back with no operand
 * loads and no epilogue, in tera-operations per second.  Blocks until done (a few milliseconds per
 * 10 000 slabs).  The measured ceiling for any int8 GEMM on the part; no counterpart in the reference. */
int b200_w8a8_selftest_mma_rate(int slabs_per_cta, double *tera_ops_per_s);

/* ---- activation quantizers ------------------------------------------------------- */

/* Per-row symmetric absmax int8 of rows of x (element type x_dtype, row stride ldx
 * elements): scales[r] = amax > 0 ? amax/127 : 1, q = clamp(rne(x/scale), -127, 127).
 * Stands in for wm_cuda_quantize_rows_f32_i8 (src/world_cuda_ops.cuh:20-21; kernel
 * src/world_cuda_ops.cu:94-125), widened to fp16/bf16 inputs and strided rows. */
int b200_w8a8_quantize_rows(const void *x, int x_dtype, int64_t ldx, int8_t *q, int64_t ldq, float *scales,
                            int rows, int cols, void *stream);

/* RMSNorm (eps) * vec_scale + vec_bias, then the quantizer above, in one pass.
 * vec_scale and vec_bias are nullable.  scale_is_mod = 1 multiplies by (1 + vec_scale[c])
 * as the reference's AdaRMSNorm does; 0 multiplies by vec_scale[c] (a plain gamma).
 * Stands in for wm_cuda_rms_norm_quantize_rows_i8 (src/world_cuda_ops.cuh:22-30; kernel
 * src/world_cuda_ops.cu:129-182). */
int b200_w8a8_rms_norm_quantize_rows(const void *x, int x_dtype, int64_t ldx, const float *vec_scale,
                                     int scale_is_mod, const float *vec_bias, int8_t *q, int64_t ldq,
                                     float *scales, int rows, int cols, float eps, void *stream);

/* v = act(float(acc) * in_row_scales[r] * w_scales[c] (+ bias[c])), then the quantizer.
 * out_row_scales may alias in_row_scales (the reference's callers do that).
 * Stands in for wm_cuda_dequant_silu_quantize_rows_i8 (src/world_cuda_ops.cuh:31-39;
 * kernel src/world_cuda_ops.cu:187-227); act selects SiLU (the reference) or GELU(tanh). */
int b200_w8a8_dequant_act_quantize_rows(const int32_t *acc, int64_t ldacc, const float *in_row_scales,
                                        const float *w_scales, const float *bias, int act, int8_t *q, int64_t ldq,
                                        float *out_row_scales, int rows, int cols, void *stream);

/* out = residual + float(acc) * row_scales[r] * col_scales[c] * (gate ? gate[c] : 1).
 * residual (nullable) has element type res_dtype, out has out_dtype; both dense [rows, cols].
 * Stands in for wm_cuda_dequant_gated_residual_f32 and wm_cuda_dequant_add_residual_f32
 * (src/world_cuda_ops.cuh:40-56; kernels src/world_cuda_ops.cu:229-262). */
int b200_w8a8_dequant_residual(const int32_t *acc, const float *row_scales, const float *col_scales,
                               const void *residual, int res_dtype, const float *gate, void *out, int out_dtype,
                               int rows, int cols, void *stream);

/* Dequantizes a QKV accumulator and applies per-head RMSNorm + 3-axis RoPE to Q and K;
 * writes head-major fp32 q[Hq,T,d], k[Hkv,T,d], v[Hkv,T,d].
 * Stands in for wm_cuda_qkv_fused_rms_rope_i32_dequant (src/world_cuda_ops.cuh:120-138;
 * kernel src/world_cuda_ops.cu:1229-1305). */
int b200_w8a8_qkv_rms_rope_dequant(const int32_t *qkv_acc, const float *row_scales, const float *weight_scales,
                                   float *q, float *k, float *v, const int64_t *x_pos, const int64_t *y_pos,
                                   const int64_t *t_pos, const float *xy, const float *inv_t, int tokens,
                                   int n_heads, int n_kv_heads, int d_head, int width, int height, float eps,
                                   void *stream);

/* ---- int8 GEMM and fused linears -------------------------------------------------- */

/* acc[m,n] = sum_k x[m,k] * w[n,k], exact int32.  x is row-major [M,K]; w is row-major
 * [N,K] (w_layout ROW_MAJOR) or SLAB128.  Needs K % 32 == 0 like the reference, and
 * 16-byte aligned x / w.  Stand in for wm_cuda_gemm_i8_i32_can_implement and
 * wm_cuda_gemm_i8_i32 (src/world_cuda_ops.cuh:315-328; src/world_cuda_ops.cu:550-599). */
int b200_w8a8_gemm_i8_i32_can_implement(const int8_t *x_i8, const int8_t *w_i8, int w_layout,
                                        const int32_t *acc_i32, int m, int k, int n);
int b200_w8a8_gemm_i8_i32(const int8_t *x_i8, const int8_t *w_i8, int w_layout, int32_t *acc_i32, int m, int k,
                          int n, void *stream);

/* Tuning aid: forces the GEMM tile width (256, 128 or 64 output columns per CTA tile) for
 * every later launch of the process; 0 restores the built-in cost model.  No counterpart in
 * the reference, whose tile shape is a compile-time template argument
 * (src/world_cuda_ops.cu:529-548). */
void b200_w8a8_set_tile_width(int bn);
/* Test aid: forces tile width (256/128/64, 0 = planner), the number of K ranges (0 = planner,
 * 1 = none) and how their partial sums meet (1 = global workspace, 2 = shared memory of a thread-block
 * cluster) for every later launch; (0, 0, 0) restores the planner.  Not thread-safe by design: set it
 * from the only thread that launches. */
void b200_w8a8_debug_force_plan(int tile_width, int k_splits, int split_mode);
/* Tuning aid: 64-wide tiles of an unsplit launch normally bring two 128-byte K slabs per copy and pipeline
 * stage (the copy engine's cost is per copy, not per byte); on = 1 keeps one slab per stage everywhere, for
 * A/B timing.  Results are identical either way. */
void b200_w8a8_debug_one_slab_stages(int on);
/* Tuning aid: 0 = the planner decides when two CTAs share one 256 x 256 tile (cta_group::2 MMA),
 * 1 = whenever the launch allows it (M > 128, unsplit 256-wide tiles, aligned buffers,
 * N % 32 == 0), 2 = never.  No counterpart in the reference. */
void b200_w8a8_set_pair_mma(int mode);
/* Switches programmatic dependent launch on (default) or off for every later launch of the
 * process.  When on, a kernel of this library may be scheduled while its predecessor in the
 * stream is still finishing, and waits on the device before it touches dependent data; off
 * gives classic full serialization, for A/B timing.  No counterpart in the reference. */
void b200_w8a8_set_overlapped_launch(int on);
/* Tuning aid, active only in a library built with -DB200_TRACE (the default build compiles the
 * timestamps out and ignores the buffer): every later GEMM launch writes nanosecond timestamps per
 * CTA (0 entry, 1 pipeline start, 2 first operands landed, 3 last MMA issued, 4 first accumulator
 * ready, 5 last epilogue done, 6 exit, 8-10 cluster split-K phases) into dev_buf[grid][16] of uint64.
 * No counterpart in the reference. */
void b200_w8a8_set_trace_buffer(void *dev_buf);

/* One fused linear: y = store( residual + gate * act( acc * x_scales[r] * w_scales[c] + bias[c] ) )
 * with bias / gate / residual nullable, y and residual of type y_dtype (fp16, bf16 or fp32)
 * with row strides ldy / ldr.  It replaces the reference's three-call sequence
 * quantized GEMM -> int32 scratch -> dequant kernel (e.g. src/world_cuda.cu:2066-2096)
 * by a GEMM whose epilogue reads the accumulator straight from tensor memory.
 * workspace: b200_w8a8_linear_workspace_size(m,k,n) bytes of device scratch (may be
 * NULL when that size is 0). */
size_t b200_w8a8_linear_workspace_size(int m, int k, int n);
int b200_w8a8_linear(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                     const float *w_scales, const float *bias, const float *gate, const void *residual,
                     int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                     void *workspace, size_t workspace_bytes, void *stream);

/* Same operation for weights that no work queued on `stream` writes (the normal case: weights
 * are uploaded once).  The kernel then requests its first weight tiles while the previous
 * kernel of the stream is still running and only waits for it before touching x, the scales,
 * the residual and y.  This is what hides the HBM latency of chained skinny linears. */
int b200_w8a8_linear_const_weights(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                                   const float *w_scales, const float *bias, const float *gate,
                                   const void *residual, int64_t ldr, void *y, int y_dtype, int64_t ldy, int m,
                                   int k, int n, int act, void *workspace, size_t workspace_bytes, void *stream);

/* A fused linear that also emits the NEXT linear's activation codes from its epilogue:
 *   y      = store( residual + gate * act( acc * x_scales[r] * w_scales[c] + bias[c] ) )   (y may be NULL)
 *   q, q_scales = per-row absmax int8 of y[:, 0:q_cols]                       (q_mode B200_RQ_PLAIN)
 *              or of RMSNorm(y[:, 0:q_cols], eps) * norm_scale + norm_bias     (q_mode B200_RQ_RMS;
 *                 norm_scale / norm_bias nullable, scale_is_mod = 1 multiplies by 1 + norm_scale)
 * computed on the values as stored in y_dtype (fp32 when y is NULL and y_dtype is fp32), so q and
 * q_scales are bit-identical to b200_w8a8_quantize_rows / b200_w8a8_rms_norm_quantize_rows run on y.
 * One launch replaces the reference's dequant kernel plus the following quantizer:
 * wm_cuda_dequant_gated_residual_f32 / wm_cuda_dequant_add_residual_f32 followed by
 * wm_cuda_rms_norm_quantize_rows_i8 (src/world_cuda.cu:2088-2120, 2146-2196, 2322-2330 with the next
 * layer's :1820-1828), wm_cuda_dequant_silu_quantize_rows_i8 (src/world_cuda_ops.cuh:31-39,
 * src/world_cuda.cu:2129-2137) and wm_cuda_quantize_rows_f32_i8 on a column block of the result.
 * A row's q_cols columns are spread over q_cols / 256 CTAs of one thread-block cluster, which
 * exchange the row statistics through distributed shared memory: that form needs q_cols a multiple
 * of 256 and at most 2048, N a multiple of 32, all buffers 16-byte aligned and ldq % 16 == 0.  Anything
 * else (the MLP hidden of 8192 columns spans 32 tiles, more than a cluster holds) runs as the linear
 * followed by the stand-alone quantizer on y -- two launches, the same codes -- and then y must be given. */
#define B200_RQ_PLAIN 1
#define B200_RQ_RMS 2
int b200_w8a8_linear_requant(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                             const float *w_scales, const float *bias, const float *gate, const void *residual,
                             int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                             int q_mode, int q_cols, const float *norm_scale, int scale_is_mod,
                             const float *norm_bias, float eps, int8_t *q, int64_t ldq, float *q_scales,
                             void *stream);
/* 0 when b200_w8a8_linear_requant runs this shape as ONE launch (buffers assumed aligned), else 1 (no message). */
int b200_w8a8_linear_requant_supported(int m, int k, int n, int q_cols);

/* The fused linear for callers that must not allocate device memory: code running under a
 * memory budget that is fixed at start-up, inside a region where the allocator may not be
 * entered (a real-time render / control loop, a callback from another runtime), or in a
 * process whose device memory is fully handed out to another framework.  It is the split-K
 * form of b200_w8a8_linear (same arguments minus the workspace, same results bit for bit);
 * its partial sums and ticket counters live in a scratch array that is part of the library
 * image: 8 MiB + 4 KiB, held on every GPU that loads the library until the process exits.
 * Limits: K >= 512, N % 4 == 0, and splits * M * N * 4 + 4096 bytes must fit the scratch
 * (b200_w8a8_linear_static_scratch_capacity()); larger shapes are rejected with a message,
 * never truncated.  It calls no cudaMalloc / cudaFree or other allocating routine.
 * The first call on each device looks up the scratch's device address
 * (cudaGetSymbolAddress); make that first call outside any stream capture.  It is also the
 * call that fixes the footprint (the library image with its scratch is resident from then on):
 * a warm-up call at start-up means no later call changes the free device memory.
 * Shapes whose planner-chosen K split would overflow the scratch run with fewer, longer K
 * ranges (down to two) before they are refused.
 * If a kernel of the library ever gives up a bounded wait, the next entry-point call that
 * reports it also re-zeroes the scratch's ticket counters (see b200_w8a8_poll_status).
 * All calls share the one scratch: two calls whose kernels can overlap on the GPU (different
 * streams, or different host threads on one device) race on it; calls on one stream are
 * safe, each launch leaves the counters zeroed for the next.
 * This entry point has no counterpart in the reference. */
size_t b200_w8a8_linear_static_scratch_capacity(void);
int b200_w8a8_linear_static_scratch(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                                    const float *w_scales, const float *bias, const float *gate,
                                    const void *residual, int64_t ldr, void *y, int y_dtype, int64_t ldy, int m,
                                    int k, int n, int act, void *stream);

/* cos / sin of every (token, rotary pair) for the positions of one frame: [tokens, d_head/2]
 * fp32 each, the values wm_cuda_qkv_fused_rms_rope_i32_dequant derives per head from the
 * frequency tables of wm_cuda_fill_rope_tables (src/world_cuda.cu:561-577).  Positions are
 * the same for every layer, so one call serves a whole pass. */
int b200_w8a8_rope_tables(const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos, const float *xy,
                          const float *inv_t, int tokens, int d_head, int width, int height, float *cos_out,
                          float *sin_out, void *stream);

/* The QKV linear with its consumer as the epilogue: int8 GEMM over
 * N = (n_heads + 2 n_kv_heads) * d_head columns, dequantized (+ bias, nullable), per-head
 * RMSNorm + rotary embedding on Q and K, written head-major fp32 q[Hq,T,d], k[Hkv,T,d],
 * v[Hkv,T,d] -- the pair wm_cuda_gemm_i8_i32 + wm_cuda_qkv_fused_rms_rope_i32_dequant
 * (src/world_cuda.cu:1840-1880; src/world_cuda_ops.cu:1229-1305) without the int32 round
 * trip, bit-identical to that pair.  d_head must be 64 (a head is two 32-column accumulator
 * loads of one thread); other head sizes use the two-call form. */
int b200_w8a8_linear_qkv_heads(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                               const float *w_scales, const float *bias, const float *rope_cos,
                               const float *rope_sin, float *q, float *k, float *v, int tokens, int k_dim,
                               int n_heads, int n_kv_heads, int d_head, float eps, void *stream);

/* Several independent skinny linears (M <= 128 rows each, own weights, own shapes) in ONE
 * launch: y_g = act(dequant(x_g @ w_g^T) + bias_g) + residual_g for every problem g.  A single
 * weight-bound linear leaves HBM idle for most of its 4-5 us of launch, first-byte and
 * hand-over latency; one persistent kernel that walks the tiles of all problems keeps the
 * weights of the next problem in flight while the current one finishes.  `problems` is a HOST
 * array (device pointers inside); w_layout, act and y_dtype are common to the group.
 * The split-K / stream-K direction the skinny shapes call for: the reference runs each such
 * linear as its own wm_cuda_gemm_i8_i32 + dequant pair (src/world_cuda.cu:2122-2153). */
typedef struct {
    const int8_t *x_i8;     /* [m, k] */
    const float *x_scales;  /* [m] */
    const int8_t *w_i8;     /* [n, k] in w_layout */
    const float *w_scales;  /* [n] */
    const float *bias;      /* [n] or NULL */
    const void *residual;   /* [m, ldr] of y_dtype or NULL */
    int64_t ldr;
    void *y;                /* [m, ldy] */
    int64_t ldy;
    int m, k, n;
} b200_w8a8_problem;
int b200_w8a8_linear_grouped(const b200_w8a8_problem *problems_host, int count, int w_layout, int act, int y_dtype,
                             void *stream);
/* Same for weights that no work queued on `stream` writes (see b200_w8a8_linear_const_weights): every CTA
 * requests the weight tiles of its first tile while the previous kernel of the stream is still draining. */
int b200_w8a8_linear_grouped_const_weights(const b200_w8a8_problem *problems_host, int count, int w_layout, int act,
                                           int y_dtype, void *stream);

/* ---- weights (HOST pointers) ------------------------------------------------------ */

/* Per-output-channel symmetric int8 quantization of host fp32 w[N,K] into `layout`,
 * using `threads` host threads (<= 0: all cores).  Rejects non-finite weights.
 * packed_host needs b200_w8a8_packed_weight_bytes(n,k,layout) bytes, scales_host n floats.
 * Stands in for copy_f32_to_i8_per_output_device (src/world_cuda.cu:153-222) minus the
 * upload, which stays with the caller. */
size_t b200_w8a8_packed_weight_bytes(int n, int k, int layout);
int b200_w8a8_pack_weight_host(const float *w_host, int n, int k, int layout, int8_t *packed_host,
                               float *scales_host, int threads);

/* ---- 128 x 128 blockwise numerics (accuracy option) -------------------------------- */

/* The rule the reference's notes name as the next step for accuracy (docs/cuda_w8a8_optimization.md:
 * 319-321 describes it, :355-356 plans it; the reference tree itself holds no implementation):
 * activations AND weights carry one scale per 128 x 128 block,
 *     scale = max(amax, 1e-8) / 128,   code = rne(v / scale) saturated to [-128, 127],
 * and the linear converts every K block's int32 partial sum to fp32 with that block pair's scales,
 *     v = 0;  for kb in order:  v = fma(float(acc_kb[r, c]), xs[r / 128][kb] * ws[c / 128][kb], v)
 * in fp32 (the scale product rounded first, one fused multiply-add per K block), followed by the epilogue
 * of b200_w8a8_linear, y = store(residual + gate * act(v + bias)) with bias / gate / residual nullable --
 * block scales inside the fused epilogues are what the reference's notes (:356) ask of this variant.
 * block_rows / x_block_rows = 128 is that rule; 1 gives every token row its own scale per K block (1 x 128
 * activation groups, scales [rows][K / 128]; weights stay 128 x 128), for inputs whose rows differ in range:
 * rows that share a 128-row block with an outlier row otherwise lose their resolution.  Scale arrays are [ceil(rows / 128)][K / 128], row-major.
 * K must be a multiple of 128; code and y buffers 16-byte aligned with 16-byte aligned rows. */
int b200_w8a8_quantize_blocks128(const void *x, int x_dtype, int64_t ldx, int8_t *q, int64_t ldq, float *block_scales,
                                 int rows, int cols, int block_rows, void *stream);
/* The Norm -> A8 fusion (b200_w8a8_rms_norm_quantize_rows) with 1 x 128 groups: (Ada)RMSNorm of each row in fp32
 * (fp64 sum of squares), then one scale per row and K block; group_scales [rows][cols / 128]; cols <= 8192. */
int b200_w8a8_rms_norm_quantize_row_blocks128(const void *x, int x_dtype, int64_t ldx, const float *vec_scale,
                                              int scale_is_mod, const float *vec_bias, int8_t *q, int64_t ldq,
                                              float *group_scales, int rows, int cols, float eps, void *stream);
int b200_w8a8_pack_weight_blocks128_host(const float *w_host, int n, int k, int layout, int8_t *packed_host,
                                         float *block_scales_host, int threads);
int b200_w8a8_linear_blocks128(const int8_t *x_i8, const float *x_block_scales, const int8_t *w_i8, int w_layout,
                               const float *w_block_scales, const float *bias, const float *gate, const void *residual,
                               int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                               int x_block_rows, void *stream);

/* ---- the linear stack (host-side driver above the operators) ----------------------- */

/* An opaque object that owns the packed int8 weights of n_layers layers plus activation
 * scratch on the current device and runs the per-layer operator sequence
 *   RMSNorm+A8 -> QKV linear -> A8 of the first d_model columns -> out linear + residual ->
 *   RMSNorm+A8 -> controller linear + residual -> RMSNorm+A8 -> up linear + GELU(tanh) ->
 *   A8 of the fp32 hidden -> down linear + residual
 * on 16-bit activations [rows, d_model].  It plays the role of the reference runtime's
 * weight upload (wm_cuda_copy_world_layers_to_device, src/world_cuda.cu:442-539), shared
 * W8A8 scratch (src/world_cuda.cu:1311-1317, 1389-1392) and layer loop
 * (world_cuda_runtime_step_rgb, src/world_cuda.cu:1819-2330) for the linears only.
 * band_rows > 0 walks the rows in bands of that height (one band through all layers of a
 * pass before the next band), which keeps a band's intermediates L2-resident.
 * Returns NULL on failure. */
void *b200_w8a8_stack_create(int d_model, int n_qkv, int d_hidden, int n_layers, int max_rows, int band_rows,
                             int act_dtype, float eps);
void b200_w8a8_stack_destroy(void *stack);
/* HOST fp32 weights [N,K] (row-major) and gammas of one layer: quantized per output
 * channel, packed to SLAB128 and uploaded; blocks until the copies are done. */
int b200_w8a8_stack_set_layer(void *stack, int layer, const float *w_qkv, const float *w_out, const float *w_ctrl,
                              const float *w_up, const float *w_down, const float *g_attn, const float *g_ctrl,
                              const float *g_mlp, int threads);
/* `steps` chained passes over all layers; x_dev is read, y_dev is written, both
 * [rows, d_model] device buffers of the stack's activation type.  use_graph = 1 captures
 * the pass once per (x_dev, y_dev, rows, steps) and replays it; it needs a real stream. */
int b200_w8a8_stack_forward(void *stack, const void *x_dev, void *y_dev, int rows, int steps, int use_graph,
                            void *stream);
/* Same with HOST buffers (pinned for full speed; use_graph = 1 bakes the two host pointers into the
 * captured graph): every band of rows is copied in, run through all layers and copied out as a
 * pipeline over two copy streams and the lanes, so the transfers of one band run under the kernels of
 * the others; returns after the whole result has landed.  The reference's runtime has the same shape at
 * its own boundary: host RGB out at the end of a step (src/world_cuda.cu:2376-2383). */
int b200_w8a8_stack_forward_host(void *stack, const void *x_host, void *y_host, int rows, int steps, int use_graph);
/* lanes = 2 runs alternate bands of rows on two streams (a second scratch set is allocated once),
 * so the bandwidth-bound quantizers of one band overlap the tensor-bound GEMMs of the other.
 * Only has an effect when a forward covers at least two bands.  The reference runs everything on
 * one stream (CMakeLists.txt:46); rows of different bands never interact, so results are
 * unchanged. */
int b200_w8a8_stack_set_lanes(void *stack, int lanes);
/* on = 1: the out, controller and down linears and the Q block of the QKV linear emit the next
 * linear's activation codes from their own epilogue (b200_w8a8_linear_requant), six launches per
 * layer; on = 0 (default): every quantizer is its own launch, ten per layer, the reference's call
 * structure (src/world_cuda.cu:1819-2330).  Results are bit-identical either way.  The fused form
 * needs d_model % 256 == 0 and d_model <= 2048; other widths always take the ten-launch form.
 * It is off by default because it measured slower on B200: a cluster of 8 CTAs fits only 15 times
 * on the 148 SMs, and the two exchanges of row statistics add more to the epilogue than the
 * separate quantizer launch costs. */
int b200_w8a8_stack_set_fusion(void *stack, int on);
/* Switches the 16-bit activation type (fp16 <-> bf16) of later forwards; both are 2 bytes,
 * so buffers are kept and only cached graphs are dropped. */
int b200_w8a8_stack_set_act_dtype(void *stack, int act_dtype);
size_t b200_w8a8_stack_device_bytes(void *stack);
/* Kernels enqueued (or replayed) by the most recent forward. */
long long b200_w8a8_stack_launches_per_forward(void *stack);

/* ---- one layer in the reference's parameterization (host-side driver above the operators) -------- */

/* Device pointers of one WorldDiT layer, owned by the caller: int8 weights [N,K] with their
 * per-channel scales and the per-layer vectors (the fields the reference keeps per layer in
 * src/world_cuda_internal.cuh:16-39 plus the modulation rows of src/world_cuda.cu:737-770).
 * w_ctrl_fc1 == NULL means the layer has no controller branch (has_ctrl, src/world_cuda.cu:2106). */
typedef struct {
    const int8_t *w_qkv;      const float *s_qkv;       /* [(Hq + 2 Hkv) * d_head, D] */
    const int8_t *w_out;      const float *s_out;       /* [D, D] */
    const int8_t *w_ctrl_fc1; const float *s_ctrl_fc1;  /* [D, D] */
    const int8_t *w_ctrl_fc2; const float *s_ctrl_fc2;  /* [D, D] */
    const int8_t *w_fc1;      const float *s_fc1;       /* [hidden, D] */
    const int8_t *w_fc2;      const float *s_fc2;       /* [D, hidden] */
    const float *mod_scale0, *mod_bias0, *gate0;        /* [D]: AdaRMSNorm before QKV (nullable), gate of the attention residual */
    const float *ctrl_cond;                             /* [D]: added before the controller's SiLU, nullable */
    const float *mod_scale1, *mod_bias1, *gate1;        /* [D]: AdaRMSNorm before the MLP (nullable), gate of the MLP residual */
} b200_w8a8_layer;

/* The W8A8 linears of one layer as two calls around the caller's attention, fp32 token stream,
 * SiLU, gated residuals, controller branch: what world_cuda_runtime_step_rgb does per layer
 * (src/world_cuda.cu:1819-1882 and 2058-2330) with each quantize -> int8 GEMM -> dequant triple
 * fused into one GEMM launch -- 13 launches per layer instead of 16 and no T x hidden int32 scratch.
 * The context owns activation scratch for up to max_tokens rows (device_bytes reports it); weights are
 * read in `w_layout` where the caller keeps them.  d_head must be 64 (see b200_w8a8_linear_qkv_heads)
 * and n_heads * d_head == d_model.  rope_cos / rope_sin come from b200_w8a8_rope_tables, once per frame.
 * tokens_next may be the same buffer as tokens. */
void *b200_w8a8_layer_ctx_create(int max_tokens, int d_model, int n_heads, int n_kv_heads, int d_head, int d_hidden,
                                 float eps, int w_layout);
void b200_w8a8_layer_ctx_destroy(void *ctx);
size_t b200_w8a8_layer_ctx_device_bytes(void *ctx);
int b200_w8a8_layer_qkv(void *ctx, const b200_w8a8_layer *layer, const float *tokens, const float *rope_cos,
                        const float *rope_sin, float *q, float *k, float *v, int n_tokens, void *stream);
int b200_w8a8_layer_after_attention(void *ctx, const b200_w8a8_layer *layer, const float *attn, const float *tokens,
                                    float *tokens_next, int n_tokens, void *stream);

/* ---- offline packed-weight file (HOST side; the writer needs no GPU) ---------------- */

/* Writes the int8 codes (slab layout) and per-channel scales of every layer, plus the three
 * norm vectors, to one file so that start-up copies bytes instead of re-quantizing fp32
 * weights.  The reference quantizes on every start (copy_f32_to_i8_per_output_device,
 * src/world_cuda.cu:153-222) and names this export as the next step of its roadmap
 * (docs/cuda_w8a8_optimization.md:357).  File: 64-byte header {magic "B2W8A8WF", version,
 * layout, d, n_qkv, hidden, layers, payload bytes, FNV-1a 64 of the payload}, then per layer
 * qkv/out/ctrl/up/down as codes + fp32 scales and g_attn/g_ctrl/g_mlp as fp32.
 * create -> add_layer x n_layers (host fp32 pointers, as stack_set_layer) -> close. */
void *b200_w8a8_weight_file_create(const char *path, int d_model, int n_qkv, int d_hidden, int n_layers);
int b200_w8a8_weight_file_add_layer(void *writer, const float *w_qkv, const float *w_out, const float *w_ctrl,
                                    const float *w_up, const float *w_down, const float *g_attn,
                                    const float *g_ctrl, const float *g_mlp, int threads);
int b200_w8a8_weight_file_close(void *writer);
/* Validates the header (and with verify != 0 the payload checksum); out-params nullable. */
int b200_w8a8_weight_file_info(const char *path, int *d_model, int *n_qkv, int *d_hidden, int *n_layers,
                               int verify);
/* Loads every layer of a stack from such a file (dimensions must match the stack's; the
 * checksum is verified first), or writes the stack's resident weights to one. */
int b200_w8a8_stack_load_weights(void *stack, const char *path);
int b200_w8a8_stack_save_weights(void *stack, const char *path);

#ifdef __cplusplus
}
#endif

#endif /* B200_W8A8_H */
