// extern "C" shells over the internal C++ interface, plus the error plumbing.
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "w8a8_internal.h"

namespace b200 {

namespace {
thread_local char t_error[512] = "";
}

int fail(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(t_error, sizeof(t_error), fmt, ap);
    va_end(ap);
    fprintf(stderr, "b200_w8a8: %s\n", t_error);
    return 1;
}

int check_launch(const char *what) {
    cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();  // clear a non-sticky launch error so the next call starts clean
        return fail("CUDA error after launching %s: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

const char *last_error_message() { return t_error; }

static bool g_pdl = true;
bool pdl_enabled() { return g_pdl; }
void set_pdl_enabled(bool on) { g_pdl = on; }

static inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

}  // namespace b200

using namespace b200;

extern "C" {

int b200_w8a8_abi_version(void) { return B200_W8A8_ABI_VERSION; }
const char *b200_w8a8_last_error(void) { return last_error_message(); }
int b200_w8a8_poll_status(int *status_out) { return status_poll(status_out); }
int b200_w8a8_selftest_mma_rate(int slabs_per_cta, double *tera_ops_per_s) {
    if (status_check_entry()) return 1;
    return mma_issue_rate(slabs_per_cta, tera_ops_per_s);
}
void b200_w8a8_debug_set_wait_limit_ns(unsigned long long ns) { set_wait_limit_ns(ns); }
void b200_w8a8_debug_drop_operand_load(int launches) { debug_drop_a_loads(launches); }
void b200_w8a8_debug_force_plan(int tile_width, int k_splits, int split_mode) {
    gemm_force_plan(tile_width, k_splits, split_mode);
}

int b200_w8a8_quantize_rows(const void *x, int x_dtype, int64_t ldx, int8_t *q, int64_t ldq, float *scales,
                            int rows, int cols, void *stream) {
    if (status_check_entry()) return 1;
    return quantize_rows(x, x_dtype, ldx, q, ldq, scales, rows, cols, as_stream(stream));
}

int b200_w8a8_rms_norm_quantize_rows(const void *x, int x_dtype, int64_t ldx, const float *vec_scale,
                                     int scale_is_mod, const float *vec_bias, int8_t *q, int64_t ldq,
                                     float *scales, int rows, int cols, float eps, void *stream) {
    if (status_check_entry()) return 1;
    return rms_norm_quantize_rows(x, x_dtype, ldx, vec_scale, scale_is_mod, vec_bias, q, ldq, scales, rows, cols,
                                  eps, as_stream(stream));
}

int b200_w8a8_dequant_act_quantize_rows(const int32_t *acc, int64_t ldacc, const float *in_row_scales,
                                        const float *w_scales, const float *bias, int act, int8_t *q, int64_t ldq,
                                        float *out_row_scales, int rows, int cols, void *stream) {
    if (status_check_entry()) return 1;
    return dequant_act_quantize_rows(acc, ldacc, in_row_scales, w_scales, bias, act, q, ldq, out_row_scales, rows,
                                     cols, as_stream(stream));
}

int b200_w8a8_dequant_residual(const int32_t *acc, const float *row_scales, const float *col_scales,
                               const void *residual, int res_dtype, const float *gate, void *out, int out_dtype,
                               int rows, int cols, void *stream) {
    if (status_check_entry()) return 1;
    return dequant_residual(acc, row_scales, col_scales, residual, res_dtype, gate, out, out_dtype, rows, cols,
                            as_stream(stream));
}

int b200_w8a8_qkv_rms_rope_dequant(const int32_t *qkv_acc, const float *row_scales, const float *weight_scales,
                                   float *q, float *k, float *v, const int64_t *x_pos, const int64_t *y_pos,
                                   const int64_t *t_pos, const float *xy, const float *inv_t, int tokens,
                                   int n_heads, int n_kv_heads, int d_head, int width, int height, float eps,
                                   void *stream) {
    if (status_check_entry()) return 1;
    return qkv_rms_rope_dequant(qkv_acc, row_scales, weight_scales, q, k, v, x_pos, y_pos, t_pos, xy, inv_t, tokens,
                                n_heads, n_kv_heads, d_head, width, height, eps, as_stream(stream));
}

int b200_w8a8_rope_tables(const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos, const float *xy,
                          const float *inv_t, int tokens, int d_head, int width, int height, float *cos_out,
                          float *sin_out, void *stream) {
    if (status_check_entry()) return 1;
    return rope_tables(x_pos, y_pos, t_pos, xy, inv_t, tokens, d_head, width, height, cos_out, sin_out,
                       as_stream(stream));
}

int b200_w8a8_linear_qkv_heads(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                               const float *w_scales, const float *bias, const float *rope_cos,
                               const float *rope_sin, float *q, float *k, float *v, int tokens, int k_dim,
                               int n_heads, int n_kv_heads, int d_head, float eps, void *stream) {
    if (status_check_entry()) return 1;
    QkvHeadsArgs a{};
    a.x = x_i8; a.row_scales = x_scales; a.w = w_i8; a.w_layout = w_layout; a.col_scales = w_scales; a.bias = bias;
    a.rope_cos = rope_cos; a.rope_sin = rope_sin; a.q = q; a.k = k; a.v = v;
    a.tokens = tokens; a.k_dim = k_dim; a.n_heads = n_heads; a.n_kv_heads = n_kv_heads; a.d_head = d_head;
    a.eps = eps;
    return linear_qkv_heads(a, as_stream(stream));
}

int b200_w8a8_linear_grouped(const b200_w8a8_problem *problems_host, int count, int w_layout, int act, int y_dtype,
                             void *stream) {
    if (status_check_entry()) return 1;
    static_assert(sizeof(b200_w8a8_problem) == sizeof(GroupedLinear), "the two problem structs share one layout");
    return linear_grouped(reinterpret_cast<const GroupedLinear *>(problems_host), count, w_layout, act, y_dtype,
                          as_stream(stream));
}

int b200_w8a8_linear_grouped_const_weights(const b200_w8a8_problem *problems_host, int count, int w_layout, int act,
                                           int y_dtype, void *stream) {
    if (status_check_entry()) return 1;
    return linear_grouped(reinterpret_cast<const GroupedLinear *>(problems_host), count, w_layout, act, y_dtype,
                          as_stream(stream), 1);
}

static LinearArgs raw_gemm_args(const int8_t *x, const int8_t *w, int w_layout, const int32_t *acc, int m, int k,
                                int n) {
    LinearArgs a{};
    a.x = x; a.w = w; a.w_layout = w_layout; a.m = m; a.k = k; a.n = n;
    a.out = const_cast<int32_t *>(acc); a.ldo = n; a.out_dtype = B200_DT_S32;
    return a;
}

int b200_w8a8_gemm_i8_i32_can_implement(const int8_t *x_i8, const int8_t *w_i8, int w_layout,
                                        const int32_t *acc_i32, int m, int k, int n) {
    return gemm_can_implement(raw_gemm_args(x_i8, w_i8, w_layout, acc_i32, m, k, n), true);
}

int b200_w8a8_gemm_i8_i32(const int8_t *x_i8, const int8_t *w_i8, int w_layout, int32_t *acc_i32, int m, int k,
                          int n, void *stream) {
    if (status_check_entry()) return 1;
    return gemm_launch(raw_gemm_args(x_i8, w_i8, w_layout, acc_i32, m, k, n), nullptr, 0, as_stream(stream));
}

void b200_w8a8_set_tile_width(int bn) { gemm_set_tile_width(bn); }
void b200_w8a8_set_pair_mma(int mode) { gemm_set_pair_mode(mode); }
void b200_w8a8_debug_one_slab_stages(int on) { gemm_set_one_slab_stages(on); }
void b200_w8a8_set_overlapped_launch(int on) { set_pdl_enabled(on != 0); }
void b200_w8a8_set_trace_buffer(void *dev_buf) { gemm_set_trace_buffer(reinterpret_cast<unsigned long long *>(dev_buf)); }

size_t b200_w8a8_linear_workspace_size(int m, int k, int n) { return gemm_workspace_size(m, k, n); }

static int linear_impl(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                       const float *w_scales, const float *bias, const float *gate, const void *residual,
                       int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                       void *workspace, size_t workspace_bytes, void *stream, int static_weights) {
    if (status_check_entry()) return 1;
    if (y_dtype == B200_DT_S32) return fail("b200_w8a8_linear writes fp16, bf16 or fp32; use gemm_i8_i32 for int32");
    LinearArgs a{};
    a.static_weights = static_weights;
    a.x = x_i8; a.w = w_i8; a.w_layout = w_layout; a.m = m; a.k = k; a.n = n;
    a.row_scales = x_scales; a.col_scales = w_scales; a.bias = bias; a.gate = gate;
    a.residual = residual; a.ldr = residual ? ldr : ldy; a.act = act;
    a.out = y; a.ldo = ldy; a.out_dtype = y_dtype;
    return gemm_launch(a, workspace, workspace_bytes, as_stream(stream));
}

int b200_w8a8_linear(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                     const float *w_scales, const float *bias, const float *gate, const void *residual,
                     int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                     void *workspace, size_t workspace_bytes, void *stream) {
    return linear_impl(x_i8, x_scales, w_i8, w_layout, w_scales, bias, gate, residual, ldr, y, y_dtype, ldy, m, k, n,
                       act, workspace, workspace_bytes, stream, 0);
}

int b200_w8a8_linear_const_weights(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                                   const float *w_scales, const float *bias, const float *gate,
                                   const void *residual, int64_t ldr, void *y, int y_dtype, int64_t ldy, int m,
                                   int k, int n, int act, void *workspace, size_t workspace_bytes, void *stream) {
    return linear_impl(x_i8, x_scales, w_i8, w_layout, w_scales, bias, gate, residual, ldr, y, y_dtype, ldy, m, k, n,
                       act, workspace, workspace_bytes, stream, 1);
}

int b200_w8a8_linear_requant(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                             const float *w_scales, const float *bias, const float *gate, const void *residual,
                             int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                             int q_mode, int q_cols, const float *norm_scale, int scale_is_mod,
                             const float *norm_bias, float eps, int8_t *q, int64_t ldq, float *q_scales,
                             void *stream) {
    if (status_check_entry()) return 1;
    LinearArgs a{};
    a.static_weights = 1;
    a.x = x_i8; a.w = w_i8; a.w_layout = w_layout; a.m = m; a.k = k; a.n = n;
    a.row_scales = x_scales; a.col_scales = w_scales; a.bias = bias; a.gate = gate;
    a.residual = residual; a.ldr = residual ? ldr : (y ? ldy : n); a.act = act;
    a.out = y; a.ldo = y ? ldy : n; a.out_dtype = y_dtype;
    RowQuantSpec qs{};
    qs.mode = q_mode; qs.cols = q_cols; qs.vec_scale = norm_scale; qs.scale_is_mod = scale_is_mod;
    qs.vec_bias = norm_bias; qs.eps = eps; qs.q = q; qs.ldq = ldq; qs.scales = q_scales;
    return linear_requant(a, qs, as_stream(stream));
}

int b200_w8a8_linear_requant_supported(int m, int k, int n, int q_cols) {
    return !(m > 0 && k > 0 && (k & 31) == 0 && n > 0 && n % 32 == 0 && q_cols > 0 && q_cols % 256 == 0 &&
             q_cols <= 2048 && q_cols <= n);
}

size_t b200_w8a8_linear_static_scratch_capacity(void) { return static_scratch_capacity(); }

int b200_w8a8_linear_static_scratch(const int8_t *x_i8, const float *x_scales, const int8_t *w_i8, int w_layout,
                                    const float *w_scales, const float *bias, const float *gate,
                                    const void *residual, int64_t ldr, void *y, int y_dtype, int64_t ldy, int m,
                                    int k, int n, int act, void *stream) {
    if (status_check_entry()) return 1;
    if (y_dtype == B200_DT_S32) return fail("b200_w8a8_linear_static_scratch writes fp16, bf16 or fp32");
    LinearArgs a{};
    a.x = x_i8; a.w = w_i8; a.w_layout = w_layout; a.m = m; a.k = k; a.n = n;
    a.row_scales = x_scales; a.col_scales = w_scales; a.bias = bias; a.gate = gate;
    a.residual = residual; a.ldr = residual ? ldr : ldy; a.act = act;
    a.out = y; a.ldo = ldy; a.out_dtype = y_dtype;
    return linear_static_scratch(a, as_stream(stream));
}

size_t b200_w8a8_packed_weight_bytes(int n, int k, int layout) { return packed_weight_bytes(n, k, layout); }

int b200_w8a8_pack_weight_host(const float *w_host, int n, int k, int layout, int8_t *packed_host,
                               float *scales_host, int threads) {
    return pack_weight_host(w_host, n, k, layout, packed_host, scales_host, threads);
}

int b200_w8a8_pack_weight_blocks128_host(const float *w_host, int n, int k, int layout, int8_t *packed_host,
                                         float *block_scales_host, int threads) {
    return pack_weight_blocks128_host(w_host, n, k, layout, packed_host, block_scales_host, threads);
}

int b200_w8a8_quantize_blocks128(const void *x, int x_dtype, int64_t ldx, int8_t *q, int64_t ldq, float *block_scales,
                                 int rows, int cols, int block_rows, void *stream) {
    if (status_check_entry()) return 1;
    if (block_rows != 128 && block_rows != 1) return fail("quantize_blocks128: block_rows must be 128 or 1, got %d", block_rows);
    return quantize_blocks128(x, x_dtype, ldx, q, ldq, block_scales, rows, cols, block_rows == 1, as_stream(stream));
}

int b200_w8a8_rms_norm_quantize_row_blocks128(const void *x, int x_dtype, int64_t ldx, const float *vec_scale,
                                              int scale_is_mod, const float *vec_bias, int8_t *q, int64_t ldq,
                                              float *group_scales, int rows, int cols, float eps, void *stream) {
    if (status_check_entry()) return 1;
    return rms_norm_quantize_row_blocks128(x, x_dtype, ldx, vec_scale, scale_is_mod, vec_bias, q, ldq, group_scales, rows,
                                           cols, eps, as_stream(stream));
}

int b200_w8a8_linear_blocks128(const int8_t *x_i8, const float *x_block_scales, const int8_t *w_i8, int w_layout,
                               const float *w_block_scales, const float *bias, const float *gate, const void *residual,
                               int64_t ldr, void *y, int y_dtype, int64_t ldy, int m, int k, int n, int act,
                               int x_block_rows, void *stream) {
    if (status_check_entry()) return 1;
    if (x_block_rows != 128 && x_block_rows != 1) return fail("linear_blocks128: x_block_rows must be 128 or 1, got %d", x_block_rows);
    Blocks128Args a = {};
    a.x = x_i8;
    a.x_scales = x_block_scales;
    a.x_scale_per_row = x_block_rows == 1;
    a.w = w_i8;
    a.w_layout = w_layout;
    a.w_scales = w_block_scales;
    a.bias = bias;
    a.gate = gate;
    a.residual = residual;
    a.ldr = ldr;
    a.act = act;
    a.out = y;
    a.ldo = ldy;
    a.out_dtype = y_dtype;
    a.m = m;
    a.k = k;
    a.n = n;
    return linear_blocks128(a, as_stream(stream));
}

}  // extern "C"
