// Definitions of the reference-named W8A8 operators (C++ linkage, no stream argument)
// on top of the C ABI.  Linking this object in place of the eight definitions in the
// reference's src/world_cuda_ops.cu makes src/world_cuda.cu call the sm_100a kernels with
// no source change.  All work goes to the per-thread default stream, which is what the
// reference's build selects for every launch (CMakeLists.txt:46).
#include <stdio.h>

#include "../../include/b200_w8a8.h"
#include "../../include/world_cuda_ops_w8a8.cuh"

int wm_cuda_quantize_rows_f32_i8(const float *x, int8_t *q, float *scales, int rows, int cols) {
    return b200_w8a8_quantize_rows(x, B200_DT_F32, cols, q, cols, scales, rows, cols, B200_STREAM_PER_THREAD);
}

int wm_cuda_rms_norm_quantize_rows_i8(const float *x, const float *mod_scale, const float *bias, int8_t *q,
                                      float *q_scales, int rows, int cols, float eps) {
    return b200_w8a8_rms_norm_quantize_rows(x, B200_DT_F32, cols, mod_scale, 1, bias, q, cols, q_scales, rows, cols,
                                            eps, B200_STREAM_PER_THREAD);
}

int wm_cuda_dequant_silu_quantize_rows_i8(const int32_t *acc, const float *input_row_scales,
                                          const float *weight_scales, const float *bias, int8_t *q,
                                          float *output_row_scales, int rows, int cols) {
    return b200_w8a8_dequant_act_quantize_rows(acc, cols, input_row_scales, weight_scales, bias, B200_ACT_SILU, q,
                                               cols, output_row_scales, rows, cols, B200_STREAM_PER_THREAD);
}

int wm_cuda_dequant_gated_residual_f32(const int32_t *acc, const float *row_scales, const float *col_scales,
                                       const float *residual, const float *gate, float *out, int rows, int cols) {
    if (!residual || !gate) {
        fprintf(stderr, "wm_cuda_dequant_gated_residual_f32: residual and gate must not be NULL\n");
        return 1;
    }
    return b200_w8a8_dequant_residual(acc, row_scales, col_scales, residual, B200_DT_F32, gate, out, B200_DT_F32,
                                      rows, cols, B200_STREAM_PER_THREAD);
}

int wm_cuda_dequant_add_residual_f32(const int32_t *acc, const float *row_scales, const float *col_scales,
                                     const float *residual, float *out, int rows, int cols) {
    if (!residual) {
        fprintf(stderr, "wm_cuda_dequant_add_residual_f32: residual must not be NULL\n");
        return 1;
    }
    return b200_w8a8_dequant_residual(acc, row_scales, col_scales, residual, B200_DT_F32, nullptr, out, B200_DT_F32,
                                      rows, cols, B200_STREAM_PER_THREAD);
}

int wm_cuda_qkv_fused_rms_rope_i32_dequant(const int32_t *qkv_acc, const float *row_scales,
                                           const float *weight_scales, float *q, float *k, float *v,
                                           const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos,
                                           const float *xy, const float *inv_t, int tokens, int n_heads,
                                           int n_kv_heads, int d_head, int width, int height, float eps) {
    return b200_w8a8_qkv_rms_rope_dequant(qkv_acc, row_scales, weight_scales, q, k, v, x_pos, y_pos, t_pos, xy, inv_t,
                                          tokens, n_heads, n_kv_heads, d_head, width, height, eps,
                                          B200_STREAM_PER_THREAD);
}

int wm_cuda_gemm_i8_i32_can_implement(const int8_t *x_i8, const int8_t *w_rm_i8, int32_t *acc_i32, int m, int k,
                                      int n) {
    return b200_w8a8_gemm_i8_i32_can_implement(x_i8, w_rm_i8, B200_W_ROW_MAJOR, acc_i32, m, k, n);
}

int wm_cuda_gemm_i8_i32(const int8_t *x_i8, const int8_t *w_rm_i8, int32_t *acc_i32, int m, int k, int n) {
    return b200_w8a8_gemm_i8_i32(x_i8, w_rm_i8, B200_W_ROW_MAJOR, acc_i32, m, k, n, B200_STREAM_PER_THREAD);
}
