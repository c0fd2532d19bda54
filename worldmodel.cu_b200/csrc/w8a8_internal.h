// Internal C++ interface shared by the translation units of the library.  The exported
// C ABI (include/b200_w8a8.h) and the reference-named operators are thin shells over this.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

#include "../../include/b200_w8a8.h"

namespace b200 {

// Records a message (stderr + thread-local buffer) and returns 1: the reference's
// operators report failure as `return 1` after printing (src/world_cuda_ops.cu:28-42).
int fail(const char *fmt, ...);
// cudaPeekAtLastError after a launch, like the reference's wm_cuda_check_launch
// (src/world_cuda_ops.cu:2856-2863).
int check_launch(const char *what);
const char *last_error_message();

// Launches with programmatic stream serialization: the kernel may begin while its predecessor
// in the stream is finishing; every kernel of the library guards its global accesses with
// griddepcontrol.wait.  pdl_enabled() can be switched off for A/B timing.
bool pdl_enabled();
void set_pdl_enabled(bool on);
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
// Same, with the grid grouped into clusters of `cluster_x` consecutive CTAs.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, unsigned cluster_x, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
    attr[1].id = cudaLaunchAttributeClusterDimension;
    attr[1].val.clusterDim.x = cluster_x;
    attr[1].val.clusterDim.y = 1;
    attr[1].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- quant_rows.cu
int quantize_rows(const void *x, int in_dtype, long long ldx, int8_t *q, long long ldq, float *scales, int rows,
                  int cols, cudaStream_t stream);
int rms_norm_quantize_rows(const void *x, int in_dtype, long long ldx, const float *vec_scale, int scale_is_mod,
                           const float *vec_bias, int8_t *q, long long ldq, float *scales, int rows, int cols,
                           float eps, cudaStream_t stream);
int dequant_act_quantize_rows(const int32_t *acc, long long ldacc, const float *in_row_scales,
                              const float *col_scales, const float *bias, int act, int8_t *q, long long ldq,
                              float *out_row_scales, int rows, int cols, cudaStream_t stream);

// ---- dequant_ops.cu
int dequant_residual(const int32_t *acc, const float *row_scales, const float *col_scales, const void *residual,
                     int res_dtype, const float *gate, void *out, int out_dtype, int rows, int cols,
                     cudaStream_t stream);
int qkv_rms_rope_dequant(const int32_t *qkv_acc, const float *row_scales, const float *weight_scales, float *q,
                         float *k, float *v, const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos,
                         const float *xy, const float *inv_t, int tokens, int n_heads, int n_kv_heads, int d_head,
                         int width, int height, float eps, cudaStream_t stream);
int rope_tables(const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos, const float *xy, const float *inv_t,
                int tokens, int d_head, int width, int height, float *cos_out, float *sin_out, cudaStream_t stream);

// ---- gemm_i8_tcgen05.cu
struct LinearArgs {
    const int8_t *x;          // A8 codes [m, k], row stride k
    const int8_t *w;          // W8 codes, row-major [n, k] or slab layout
    int w_layout;             // B200_W_ROW_MAJOR / B200_W_SLAB128
    int m, k, n;
    // epilogue (all nullable except out)
    const float *row_scales;  // [m]
    const float *col_scales;  // [n]
    const float *bias;        // [n]
    const float *gate;        // [n]
    const void *residual;     // [m, ldr] in out dtype
    long long ldr;
    int act;
    void *out;                // [m, ldo]
    long long ldo;
    int out_dtype;            // B200_DT_S32 means raw accumulators, epilogue inputs ignored
    int static_weights;       // w is never written by work queued on the stream: its first tiles may be
                              // fetched before the predecessor kernel has finished
};
// QKV linear with the per-head RMSNorm + rotary consumer as its epilogue (d_head = 64).
struct QkvHeadsArgs {
    const int8_t *x;          // A8 codes [tokens, k_dim]
    const int8_t *w;          // W8 codes [(Hq + 2 Hkv) * 64, k_dim], row-major or slab layout
    int w_layout;
    const float *row_scales;  // [tokens]
    const float *col_scales;  // [(Hq + 2 Hkv) * 64]
    const float *bias;        // nullable
    const float *rope_cos;    // [tokens, 32]
    const float *rope_sin;    // [tokens, 32]
    float *q, *k, *v;         // head-major fp32 [Hq,T,64], [Hkv,T,64], [Hkv,T,64]
    int tokens, k_dim, n_heads, n_kv_heads, d_head;
    float eps;
    int static_weights;
};
int linear_qkv_heads(const QkvHeadsArgs &q, cudaStream_t stream);
// ---- gemm_i8_rowq.cu: a linear whose epilogue also quantizes the first `cols` columns of its
// result per row (optionally RMS-normalised first) into the next linear's A8 codes.
struct RowQuantSpec {
    int mode;                // B200_RQ_PLAIN / B200_RQ_RMS
    int cols;                // quantized width: a multiple of 256, at most 2048, at most N
    const float *vec_scale;  // RMS mode: gamma or modulation [cols], nullable
    int scale_is_mod;        // 1: multiply by (1 + vec_scale)
    const float *vec_bias;   // RMS mode: [cols], nullable
    float eps;
    int8_t *q;               // [m, ldq] codes
    long long ldq;
    float *scales;           // [m]
};
// nullptr when the fused form can run these arguments, else the reason it cannot
const char *linear_requant_unsupported(const LinearArgs &a, const RowQuantSpec &qs);
// a.out may be null (codes only); a.out_dtype then still names the type the value is rounded to
int linear_requant(const LinearArgs &a, const RowQuantSpec &qs, cudaStream_t stream);
// One of several independent skinny linears (M <= 128) run by a single launch; the exported
// b200_w8a8_problem has the same fields in the same order.
struct GroupedLinear {
    const int8_t *x;          // A8 codes [m, k]
    const float *row_scales;  // [m]
    const int8_t *w;          // W8 codes in the layout of the call
    const float *col_scales;  // [n]
    const float *bias;        // [n], nullable
    const void *residual;     // [m, ldr] in the output type, nullable
    long long ldr;
    void *out;                // [m, ldo]
    long long ldo;
    int m, k, n;
};
int linear_grouped(const GroupedLinear *problems, int count, int w_layout, int act, int out_dtype,
                   cudaStream_t stream, int static_weights = 0);
int gemm_can_implement(const LinearArgs &a, bool verbose);
int gemm_launch(const LinearArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream);
size_t gemm_workspace_size(int m, int k, int n);
void gemm_reset_static_tickets();

// ---- gemm_i8_blocks128.cu: the 128 x 128 blockwise numerics (one scale per block of activations and of weights,
// scale = max(amax, 1e-8) / 128, codes in [-128, 127], fp32 accumulation K block by K block)
struct Blocks128Args {
    const int8_t *x;         // codes [m, k], row stride k
    const float *x_scales;   // [ceil(m / 128)][k / 128], or [m][k / 128] with x_scale_per_row
    int x_scale_per_row;     // activations quantized in 1 x 128 groups (a scale per row and K block)
    const int8_t *w;         // codes, row-major [n, k] or slab layout
    int w_layout;
    const float *w_scales;   // [ceil(n / 128)][k / 128]
    const float *bias;       // [n], nullable
    const float *gate;       // [n], nullable
    const void *residual;    // [m, ldr] in the output type, nullable
    long long ldr;
    int act;
    void *out;               // [m, ldo]
    long long ldo;
    int out_dtype;           // fp32, fp16 or bf16
    int m, k, n;
};
int quantize_blocks128(const void *x, int in_dtype, long long ldx, int8_t *q, long long ldq, float *scales, int rows,
                       int cols, int per_row, cudaStream_t stream);
int linear_blocks128(const Blocks128Args &a, cudaStream_t stream);
int rms_norm_quantize_row_blocks128(const void *x, int in_dtype, long long ldx, const float *vec_scale, int scale_is_mod,
                                    const float *vec_bias, int8_t *q, long long ldq, float *scales, int rows, int cols,
                                    float eps, cudaStream_t stream);

// ---- status.cu
// Device-visible address of the status word (pinned host memory mapped into the device when
// may_allocate allows creating it, else a __device__ variable).
int *status_slot(bool may_allocate);
unsigned long long wait_limit_ns();
void set_wait_limit_ns(unsigned long long ns);
void debug_drop_a_loads(int launches);
int take_debug_drop();
// Plain host load of the mapped status word: non-zero means an earlier kernel gave up a wait;
// reports it (return 1, message), clears it and re-zeroes the library's own split-K tickets.
int status_check_entry();
int status_poll(int *status_out);
int linear_static_scratch(const LinearArgs &a, cudaStream_t stream);
size_t static_scratch_capacity();
void gemm_set_tile_width(int bn);
void gemm_set_pair_mode(int mode);
void gemm_set_one_slab_stages(int on);
void gemm_set_trace_buffer(unsigned long long *dev_buf);
unsigned long long *gemm_trace_buffer();
void gemm_force_plan(int bn, int splits, int mode);
int gemm_forced_tile_width();  // 0 unless a test forced one

// ---- mma_rate.cu
int mma_issue_rate(int slabs_per_cta, double *tera_ops_per_s);

// ---- pack_weights.cpp
int pack_weight_host(const float *w, int n, int k, int layout, int8_t *packed, float *scales, int threads);
size_t packed_weight_bytes(int n, int k, int layout);
int pack_weight_blocks128_host(const float *w, int n, int k, int layout, int8_t *packed, float *scales, int threads);

// ---- weight_file.cpp (host only)
struct WeightFileWriter;
size_t weight_file_layer_bytes(int d, int n_qkv, int hidden);
WeightFileWriter *weight_file_create(const char *path, int d, int n_qkv, int hidden, int n_layers);
int weight_file_add_packed(WeightFileWriter *w, const int8_t *const codes[5], const float *const scales[5],
                           const float *const gammas[3]);
int weight_file_close(WeightFileWriter *w);
int weight_file_info(const char *path, int *d, int *n_qkv, int *hidden, int *n_layers, int verify);
int weight_file_read_layer(const char *path, int layer, int d, int n_qkv, int hidden, void *dst);

}  // namespace b200
