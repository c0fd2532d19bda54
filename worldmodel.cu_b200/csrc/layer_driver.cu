// One WorldDiT layer's W8A8 linears in the reference's own parameterization, as two calls around
// the caller's attention.  It is the step driver of the reference with the operator triples
// fused: where world_cuda_runtime_step_rgb issues quantize -> int8 GEMM -> dequant kernel
// (src/world_cuda.cu:1819-1882, 2058-2096, 2107-2154, 2187-2330: sixteen launches per layer and a
// T x hidden int32 scratch that is written and re-read six times), this issues
//
//   b200_w8a8_layer_qkv:              AdaRMSNorm(mod_scale0, mod_bias0) -> A8
//                                     QKV linear with per-head RMSNorm + RoPE epilogue -> q, k, v head-major
//   [attention: the caller's]
//   b200_w8a8_layer_after_attention:  A8(attn) -> out linear * gate0 + tokens            -> x_a
//                                     RMSNorm -> A8 -> ctrl fc1 + cond, SiLU (fp32) -> A8
//                                                   -> ctrl fc2 + x_a                    -> x_c   (layers with a controller)
//                                     AdaRMSNorm(mod_scale1, mod_bias1) -> A8 -> fc1, SiLU (fp32) -> A8
//                                                   -> fc2 * gate1 + x_c                 -> next tokens
//
// thirteen launches, no int32 scratch, fp32 token stream like the reference.  Weights stay where the
// caller put them (row-major int8 [N,K] as copy_f32_to_i8_per_output_device uploads them,
// src/world_cuda.cu:153-222, or the slab layout); the context only owns activation scratch.
#include <stdio.h>

#include "w8a8_internal.h"

namespace b200 {
namespace {

struct LayerCtx {
    int max_tokens = 0, d = 0, n_heads = 0, n_kv_heads = 0, d_head = 0, n_qkv = 0, hidden = 0, w_layout = 0;
    float eps = 0.0f;
    int8_t *a8 = nullptr;       // [T, max(d, hidden)]
    float *a8_scales = nullptr; // [T]
    float *h = nullptr;         // [T, hidden] fp32 hidden before re-quantization (also the controller's [T, d])
    float *xa = nullptr, *xc = nullptr;  // [T, d] token stream after attention / after the controller
    size_t bytes = 0;
};

int ctx_alloc(LayerCtx *c, void **p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) return fail("cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
    c->bytes += bytes;
    return 0;
}

int run_linear(const LayerCtx *c, const int8_t *w, const float *sw, int n, int k, const float *bias, const float *gate,
               const float *residual, int act, float *out, int rows, cudaStream_t st) {
    LinearArgs a{};
    a.x = c->a8; a.w = w; a.w_layout = c->w_layout; a.m = rows; a.k = k; a.n = n;
    a.row_scales = c->a8_scales; a.col_scales = sw; a.bias = bias; a.gate = gate;
    a.residual = residual; a.ldr = n; a.act = act;
    a.out = out; a.ldo = n; a.out_dtype = B200_DT_F32;
    a.static_weights = 1;  // weights are uploaded once, before any step
    return gemm_launch(a, nullptr, 0, st);
}

}  // namespace
}  // namespace b200

using namespace b200;

extern "C" {

void b200_w8a8_layer_ctx_destroy(void *handle) {
    LayerCtx *c = reinterpret_cast<LayerCtx *>(handle);
    if (!c) return;
    cudaFree(c->a8);
    cudaFree(c->a8_scales);
    cudaFree(c->h);
    cudaFree(c->xa);
    cudaFree(c->xc);
    delete c;
}

void *b200_w8a8_layer_ctx_create(int max_tokens, int d_model, int n_heads, int n_kv_heads, int d_head, int d_hidden,
                                 float eps, int w_layout) {
    if (max_tokens <= 0 || d_model <= 0 || n_heads <= 0 || n_kv_heads <= 0 || d_head <= 0 || d_hidden <= 0 ||
        n_heads * d_head != d_model || d_model % 32 != 0 || d_hidden % 32 != 0 ||
        (w_layout != B200_W_ROW_MAJOR && w_layout != B200_W_SLAB128)) {
        fail("invalid layer context tokens=%d d=%d heads=%d/%d d_head=%d hidden=%d layout=%d (needs heads * d_head == d)",
             max_tokens, d_model, n_heads, n_kv_heads, d_head, d_hidden, w_layout);
        return nullptr;
    }
    status_slot(true);
    LayerCtx *c = new LayerCtx();
    c->max_tokens = max_tokens; c->d = d_model; c->n_heads = n_heads; c->n_kv_heads = n_kv_heads; c->d_head = d_head;
    c->n_qkv = (n_heads + 2 * n_kv_heads) * d_head; c->hidden = d_hidden; c->eps = eps; c->w_layout = w_layout;
    const size_t T = (size_t)max_tokens, wide = (size_t)(d_hidden > d_model ? d_hidden : d_model);
    if (ctx_alloc(c, (void **)&c->a8, T * wide) || ctx_alloc(c, (void **)&c->a8_scales, T * sizeof(float)) ||
        ctx_alloc(c, (void **)&c->h, T * wide * sizeof(float)) || ctx_alloc(c, (void **)&c->xa, T * d_model * sizeof(float)) ||
        ctx_alloc(c, (void **)&c->xc, T * d_model * sizeof(float))) {
        b200_w8a8_layer_ctx_destroy(c);
        return nullptr;
    }
    return c;
}

size_t b200_w8a8_layer_ctx_device_bytes(void *handle) {
    LayerCtx *c = reinterpret_cast<LayerCtx *>(handle);
    return c ? c->bytes : 0;
}

int b200_w8a8_layer_qkv(void *handle, const b200_w8a8_layer *L, const float *tokens, const float *rope_cos,
                        const float *rope_sin, float *q, float *k, float *v, int n_tokens, void *stream) {
    LayerCtx *c = reinterpret_cast<LayerCtx *>(handle);
    if (status_check_entry()) return 1;
    if (!c || !L || !tokens || !rope_cos || !rope_sin || !q || !k || !v || n_tokens <= 0 || n_tokens > c->max_tokens ||
        !L->w_qkv || !L->s_qkv)
        return fail("invalid layer_qkv arguments (tokens=%d)", n_tokens);
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    if (rms_norm_quantize_rows(tokens, B200_DT_F32, c->d, L->mod_scale0, 1, L->mod_bias0, c->a8, c->d, c->a8_scales,
                               n_tokens, c->d, c->eps, st))
        return 1;
    QkvHeadsArgs a{};
    a.x = c->a8; a.row_scales = c->a8_scales; a.w = L->w_qkv; a.w_layout = c->w_layout; a.col_scales = L->s_qkv;
    a.rope_cos = rope_cos; a.rope_sin = rope_sin; a.q = q; a.k = k; a.v = v;
    a.tokens = n_tokens; a.k_dim = c->d; a.n_heads = c->n_heads; a.n_kv_heads = c->n_kv_heads; a.d_head = c->d_head;
    a.eps = c->eps; a.static_weights = 1;
    return linear_qkv_heads(a, st);
}

int b200_w8a8_layer_after_attention(void *handle, const b200_w8a8_layer *L, const float *attn, const float *tokens,
                                    float *tokens_next, int n_tokens, void *stream) {
    LayerCtx *c = reinterpret_cast<LayerCtx *>(handle);
    if (status_check_entry()) return 1;
    if (!c || !L || !attn || !tokens || !tokens_next || n_tokens <= 0 || n_tokens > c->max_tokens || !L->w_out ||
        !L->s_out || !L->gate0 || !L->w_fc1 || !L->s_fc1 || !L->w_fc2 || !L->s_fc2 || !L->gate1)
        return fail("invalid layer_after_attention arguments (tokens=%d)", n_tokens);
    const bool ctrl = L->w_ctrl_fc1 != nullptr;
    if (ctrl && (!L->s_ctrl_fc1 || !L->w_ctrl_fc2 || !L->s_ctrl_fc2))
        return fail("layer_after_attention: a controller branch needs both of its linears and their scales");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
    const int T = n_tokens, d = c->d, hid = c->hidden;
    // attention output -> out projection, gated, onto the token stream (src/world_cuda.cu:2058-2096)
    if (quantize_rows(attn, B200_DT_F32, d, c->a8, d, c->a8_scales, T, d, st)) return 1;
    if (run_linear(c, L->w_out, L->s_out, d, d, nullptr, L->gate0, tokens, B200_ACT_NONE, c->xa, T, st)) return 1;
    const float *x_mlp = c->xa;
    if (ctrl) {
        // controller branch: RMSNorm -> fc1 + cond -> SiLU -> fc2, added back (src/world_cuda.cu:2107-2154)
        if (rms_norm_quantize_rows(c->xa, B200_DT_F32, d, nullptr, 0, nullptr, c->a8, d, c->a8_scales, T, d, c->eps, st))
            return 1;
        if (run_linear(c, L->w_ctrl_fc1, L->s_ctrl_fc1, d, d, L->ctrl_cond, nullptr, nullptr, B200_ACT_SILU, c->h, T, st))
            return 1;
        if (quantize_rows(c->h, B200_DT_F32, d, c->a8, d, c->a8_scales, T, d, st)) return 1;
        if (run_linear(c, L->w_ctrl_fc2, L->s_ctrl_fc2, d, d, nullptr, nullptr, c->xa, B200_ACT_NONE, c->xc, T, st))
            return 1;
        x_mlp = c->xc;
    }
    // MLP: AdaRMSNorm -> fc1 -> SiLU -> fc2, gated, onto the stream (src/world_cuda.cu:2187-2330)
    if (rms_norm_quantize_rows(x_mlp, B200_DT_F32, d, L->mod_scale1, 1, L->mod_bias1, c->a8, d, c->a8_scales, T, d,
                               c->eps, st))
        return 1;
    if (run_linear(c, L->w_fc1, L->s_fc1, hid, d, nullptr, nullptr, nullptr, B200_ACT_SILU, c->h, T, st)) return 1;
    if (quantize_rows(c->h, B200_DT_F32, hid, c->a8, hid, c->a8_scales, T, hid, st)) return 1;
    return run_linear(c, L->w_fc2, L->s_fc2, d, hid, nullptr, L->gate1, x_mlp, B200_ACT_NONE, tokens_next, T, st);
}

}  // extern "C"
