// Host-side driver of the W8A8 linear stack: owns the packed int8 weights of every layer
// and the activation scratch, and enqueues one denoising pass (layers x the ten operators
// of a layer) on a stream, optionally replayed as a CUDA graph.
//
// It is the part of the reference's runtime that sits directly above the operators,
// restricted to the linears: weight quantization + upload
// (wm_cuda_copy_world_layers_to_device, src/world_cuda.cu:442-539), shared scratch
// (src/world_cuda.cu:1311-1317, 1389-1392) and the per-layer call sequence
// (world_cuda_runtime_step_rgb, src/world_cuda.cu:1819-2330) with attention left out.
// Differences by design: the int32 scratch is gone (epilogues read tensor memory), the
// controller linear is a residual branch, activations are 16-bit, and rows can be walked
// in bands so a band's intermediates stay in L2 between producer and consumer kernels.
#include <stdint.h>
#include <stdio.h>

#include <map>
#include <tuple>
#include <vector>

#include "w8a8_internal.h"

namespace b200 {

namespace {

struct Weight {
    int8_t *codes = nullptr;
    float *scales = nullptr;
    int n = 0, k = 0;
};

struct Layer {
    Weight qkv, out, ctrl, up, down;
    float *g_attn = nullptr, *g_ctrl = nullptr, *g_mlp = nullptr;
    bool loaded = false;
};

}  // namespace

struct Stack {
    int d = 0, n_qkv = 0, hidden = 0, n_layers = 0, max_rows = 0, band_rows = 0, dtype = B200_DT_F16;
    float eps = 1e-6f;
    int device = 0;
    std::vector<Layer> layers;
    // full-height token buffers (residual stream) and band-height scratch
    void *tok[3] = {nullptr, nullptr, nullptr};
    // band-height scratch, one set per lane: bands are independent (rows never interact), so two
    // lanes on two streams let one band's bandwidth-bound quantizers run under the other band's GEMMs
    struct Scratch {
        int8_t *a8 = nullptr;        // [band, max(d, hidden)]
        float *a8_scales = nullptr;  // [band]
        int8_t *a8_alt = nullptr;    // second code buffer: a linear that emits the next linear's codes
        float *a8_alt_scales = nullptr;  // cannot write them over the codes it is still reading
        void *qkv = nullptr;         // [band, n_qkv] 16-bit
        float *h = nullptr;          // [band, hidden] fp32 hidden before re-quantization
    } scratch[2];
    int lanes = 1;
    int fusion = 0;      // 1: linears with d_model output columns emit the next linear's codes from their epilogue
                         // (off by default: measured slower on B200 at every row count, see stack_set_fusion)
    bool fuse_ok = false;  // the shapes allow it (d_model a multiple of 256, at most 2048)
    cudaStream_t lane_stream = nullptr;   // stream of the second lane
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    // host entry point: bands are copied in, computed and copied out as a pipeline
    cudaStream_t copy_in_stream = nullptr, copy_out_stream = nullptr;
    cudaEvent_t ev_copy_fork = nullptr, ev_copy_join = nullptr;
    std::vector<cudaEvent_t> ev_band_in, ev_band_done;
    std::map<std::tuple<const void *, void *, int, int>, cudaGraphExec_t> host_graphs;
    void *host_stage = nullptr; // device staging for the host entry point
    void *host_out = nullptr;
    cudaStream_t own_stream = nullptr;
    size_t device_bytes = 0;
    std::map<std::tuple<const void *, void *, int, int>, cudaGraphExec_t> graphs;
    long long launches_per_forward = 0;
};

namespace {

size_t esize(int dtype) { return dtype == B200_DT_F32 ? 4 : 2; }

int dev_alloc(Stack *s, void **p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes);
    if (e != cudaSuccess) return fail("cudaMalloc(%zu bytes): %s", bytes, cudaGetErrorString(e));
    s->device_bytes += bytes;
    return 0;
}

int upload_weight(Stack *s, Weight *w, const float *host, int n, int k, int threads) {
    std::vector<int8_t> packed(packed_weight_bytes(n, k, B200_W_SLAB128));
    std::vector<float> scales((size_t)n);
    if (pack_weight_host(host, n, k, B200_W_SLAB128, packed.data(), scales.data(), threads)) return 1;
    if (!w->codes) {
        if (dev_alloc(s, (void **)&w->codes, packed.size())) return 1;
        if (dev_alloc(s, (void **)&w->scales, (size_t)n * sizeof(float))) return 1;
    }
    w->n = n;
    w->k = k;
    cudaError_t e = cudaMemcpy(w->codes, packed.data(), packed.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w->scales, scales.data(), (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail("CUDA error while copying W8 weights [%d,%d]: %s", n, k, cudaGetErrorString(e));
    return 0;
}

int upload_vec(Stack *s, float **dst, const float *host, int n) {
    if (!*dst && dev_alloc(s, (void **)dst, (size_t)n * sizeof(float))) return 1;
    cudaError_t e = cudaMemcpy(*dst, host, (size_t)n * sizeof(float), cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail("CUDA error while copying a norm vector: %s", cudaGetErrorString(e));
    return 0;
}

int fused(const Stack *s, const Weight &w, const int8_t *a8, const float *a8_scales, const void *residual, int act,
          void *out, int out_dtype, long long ldo, int rows, cudaStream_t stream) {
    LinearArgs a{};
    a.x = a8; a.w = w.codes; a.w_layout = B200_W_SLAB128; a.m = rows; a.k = w.k; a.n = w.n;
    a.row_scales = a8_scales; a.col_scales = w.scales; a.residual = residual; a.ldr = w.n; a.act = act;
    a.out = out; a.ldo = ldo; a.out_dtype = out_dtype;
    a.static_weights = 1;  // the stack's weights are written only by set_layer, which blocks
    return gemm_launch(a, nullptr, 0, stream);
}

// A fused linear that also emits the codes of the next linear's input (its first d columns,
// RMS-normalised with `gamma` when given) into q_out / s_out.
int fused_requant(const Stack *s, const Weight &w, const int8_t *a8, const float *a8_scales, const void *residual,
                  void *out, long long ldo, const float *gamma, int8_t *q_out, float *s_out, int rows,
                  cudaStream_t stream) {
    LinearArgs a{};
    a.x = a8; a.w = w.codes; a.w_layout = B200_W_SLAB128; a.m = rows; a.k = w.k; a.n = w.n;
    a.row_scales = a8_scales; a.col_scales = w.scales; a.residual = residual; a.ldr = w.n; a.act = B200_ACT_NONE;
    a.out = out; a.ldo = ldo; a.out_dtype = s->dtype;
    a.static_weights = 1;
    RowQuantSpec qs{};
    qs.mode = gamma ? B200_RQ_RMS : B200_RQ_PLAIN;
    qs.cols = s->d; qs.vec_scale = gamma; qs.scale_is_mod = 0; qs.vec_bias = nullptr; qs.eps = s->eps;
    qs.q = q_out; qs.ldq = s->d; qs.scales = s_out;
    return linear_requant(a, qs, stream);
}

// One layer with the four quantizers that follow a linear folded into that linear: six launches
// instead of ten.  `have_codes` says that the previous layer's down projection already left the
// RMS-normalised codes of x in the scratch; `next_gamma` (null for the very last layer) is the
// first norm vector of the layer that follows.  The two code buffers alternate: *cur names the
// one that holds the current linear's input.
int layer_band_fused(Stack *s, const Stack::Scratch &w, const Layer &L, const void *x, void *x1, void *x2, void *x3,
                     int rows, bool have_codes, const float *next_gamma, int *cur, long long *launches,
                     cudaStream_t st) {
    const int d = s->d, dt = s->dtype;
    int8_t *qb[2] = {w.a8, w.a8_alt};
    float *sb[2] = {w.a8_scales, w.a8_alt_scales};
    int c = *cur;
    if (!have_codes) {
        if (rms_norm_quantize_rows(x, dt, d, L.g_attn, 0, nullptr, qb[c], d, sb[c], rows, d, s->eps, st)) return 1;
        ++*launches;
    }
    if (fused_requant(s, L.qkv, qb[c], sb[c], nullptr, w.qkv, s->n_qkv, nullptr, qb[c ^ 1], sb[c ^ 1], rows, st)) return 1;
    c ^= 1;
    if (fused_requant(s, L.out, qb[c], sb[c], x, x1, d, L.g_ctrl, qb[c ^ 1], sb[c ^ 1], rows, st)) return 1;
    c ^= 1;
    if (fused_requant(s, L.ctrl, qb[c], sb[c], x1, x2, d, L.g_mlp, qb[c ^ 1], sb[c ^ 1], rows, st)) return 1;
    c ^= 1;
    if (fused(s, L.up, qb[c], sb[c], nullptr, B200_ACT_GELU_TANH, w.h, B200_DT_F32, s->hidden, rows, st)) return 1;
    if (quantize_rows(w.h, B200_DT_F32, s->hidden, qb[c], s->hidden, sb[c], rows, s->hidden, st)) return 1;
    if (next_gamma) {
        if (fused_requant(s, L.down, qb[c], sb[c], x2, x3, d, next_gamma, qb[c ^ 1], sb[c ^ 1], rows, st)) return 1;
        c ^= 1;
    } else {
        if (fused(s, L.down, qb[c], sb[c], x2, B200_ACT_NONE, x3, dt, d, rows, st)) return 1;
    }
    *launches += 6;
    *cur = c;
    return 0;
}

// The ten operators of one layer on one band of rows of the residual stream.
int layer_band(Stack *s, const Stack::Scratch &w, const Layer &L, const void *x, void *x1, void *x2, void *x3,
               int rows, cudaStream_t st) {
    const int d = s->d, dt = s->dtype;
    if (rms_norm_quantize_rows(x, dt, d, L.g_attn, 0, nullptr, w.a8, d, w.a8_scales, rows, d, s->eps, st)) return 1;
    if (fused(s, L.qkv, w.a8, w.a8_scales, nullptr, B200_ACT_NONE, w.qkv, dt, s->n_qkv, rows, st)) return 1;
    if (quantize_rows(w.qkv, dt, s->n_qkv, w.a8, d, w.a8_scales, rows, d, st)) return 1;
    if (fused(s, L.out, w.a8, w.a8_scales, x, B200_ACT_NONE, x1, dt, d, rows, st)) return 1;
    if (rms_norm_quantize_rows(x1, dt, d, L.g_ctrl, 0, nullptr, w.a8, d, w.a8_scales, rows, d, s->eps, st)) return 1;
    if (fused(s, L.ctrl, w.a8, w.a8_scales, x1, B200_ACT_NONE, x2, dt, d, rows, st)) return 1;
    if (rms_norm_quantize_rows(x2, dt, d, L.g_mlp, 0, nullptr, w.a8, d, w.a8_scales, rows, d, s->eps, st)) return 1;
    if (fused(s, L.up, w.a8, w.a8_scales, nullptr, B200_ACT_GELU_TANH, w.h, B200_DT_F32, s->hidden, rows, st))
        return 1;
    if (quantize_rows(w.h, B200_DT_F32, s->hidden, w.a8, s->hidden, w.a8_scales, rows, s->hidden, st)) return 1;
    if (fused(s, L.down, w.a8, w.a8_scales, x2, B200_ACT_NONE, x3, dt, d, rows, st)) return 1;
    return 0;
}

// Streams and events of the copy pipeline of the host entry point, created on first use.
int ensure_copy_pipeline(Stack *s, int n_bands) {
    if (!s->copy_in_stream) {
        if (cudaStreamCreateWithFlags(&s->copy_in_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaStreamCreateWithFlags(&s->copy_out_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->ev_copy_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->ev_copy_join, cudaEventDisableTiming) != cudaSuccess)
            return fail("creating the copy streams failed");
    }
    while ((int)s->ev_band_in.size() < n_bands) {
        cudaEvent_t a = nullptr, b = nullptr;
        if (cudaEventCreateWithFlags(&a, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&b, cudaEventDisableTiming) != cudaSuccess)
            return fail("creating the band events failed");
        s->ev_band_in.push_back(a);
        s->ev_band_done.push_back(b);
    }
    return 0;
}

// Enqueues `steps` passes over `rows` rows.  With x_host / y_host given (the host entry point) every band's
// rows are copied in on a copy stream before that band's kernels and copied out on another after them, so
// that the transfers of one band run under the kernels of the others; x and y are then device staging.
int enqueue(Stack *s, const void *x, void *y, int rows, int steps, cudaStream_t st, const void *x_host = nullptr,
            void *y_host = nullptr) {
    const size_t row_bytes = (size_t)s->d * esize(s->dtype);
    const int total_layers = steps * s->n_layers;
    long long launches = 0;
    const int n_bands = (rows + s->band_rows - 1) / s->band_rows;
    const bool two_lanes = s->lanes == 2 && n_bands >= 2;
    const bool piped = x_host != nullptr;
    if (two_lanes) {  // the second lane starts after everything already queued on the caller's stream
        if (cudaEventRecord(s->ev_fork, st) != cudaSuccess ||
            cudaStreamWaitEvent(s->lane_stream, s->ev_fork, 0) != cudaSuccess)
            return fail("forking the second lane failed");
    }
    if (piped) {
        if (ensure_copy_pipeline(s, n_bands)) return 1;
        if (cudaEventRecord(s->ev_copy_fork, st) != cudaSuccess ||
            cudaStreamWaitEvent(s->copy_in_stream, s->ev_copy_fork, 0) != cudaSuccess ||
            cudaStreamWaitEvent(s->copy_out_stream, s->ev_copy_fork, 0) != cudaSuccess)
            return fail("forking the copy streams failed");
        int b = 0;
        for (int r0 = 0; r0 < rows; r0 += s->band_rows, ++b) {
            const int nr = rows - r0 < s->band_rows ? rows - r0 : s->band_rows;
            const size_t off = (size_t)r0 * row_bytes;
            if (cudaMemcpyAsync((char *)const_cast<void *>(x) + off, (const char *)x_host + off, (size_t)nr * row_bytes,
                                cudaMemcpyHostToDevice, s->copy_in_stream) != cudaSuccess ||
                cudaEventRecord(s->ev_band_in[b], s->copy_in_stream) != cudaSuccess)
                return fail("queueing the H2D copy of band %d failed", b);
        }
    }
    int band = 0;
    for (int r0 = 0; r0 < rows; r0 += s->band_rows, ++band) {
        const int nr = rows - r0 < s->band_rows ? rows - r0 : s->band_rows;
        const int lane = two_lanes ? (band & 1) : 0;
        cudaStream_t bst = lane ? s->lane_stream : st;
        const Stack::Scratch &w = s->scratch[lane];
        const size_t off = (size_t)r0 * row_bytes;
        if (piped && cudaStreamWaitEvent(bst, s->ev_band_in[band], 0) != cudaSuccess)
            return fail("waiting for the H2D copy of band %d failed", band);
        const void *cur = (const char *)x + off;
        int cur_slot = -1;  // -1: caller's input
        const bool fuse = s->fusion && s->fuse_ok;
        int code_buf = 0;
        for (int li = 0; li < total_layers; ++li) {
            const Layer &L = s->layers[li % s->n_layers];
            // Three internal buffers rotate.  x is dead once x1 exists (it is read by the
            // first norm and as the residual of the out projection only), so the layer's
            // result x3 may take x's buffer; the caller's input buffer is never written.
            int free_slots[3], nf = 0;
            for (int i = 0; i < 3; ++i)
                if (i != cur_slot) free_slots[nf++] = i;
            void *x1 = (char *)s->tok[free_slots[0]] + off;
            void *x2 = (char *)s->tok[free_slots[1]] + off;
            const int x3_slot = cur_slot >= 0 ? cur_slot : free_slots[2];
            const bool last = li == total_layers - 1;
            void *x3 = last ? (char *)y + off : (char *)s->tok[x3_slot] + off;
            if (fuse) {
                const float *next_gamma = last ? nullptr : s->layers[(li + 1) % s->n_layers].g_attn;
                if (layer_band_fused(s, w, L, cur, x1, x2, x3, nr, li > 0, next_gamma, &code_buf, &launches, bst)) return 1;
            } else {
                if (layer_band(s, w, L, cur, x1, x2, x3, nr, bst)) return 1;
                launches += 10;
            }
            cur = x3;
            cur_slot = x3_slot;
        }
        if (piped) {
            if (cudaEventRecord(s->ev_band_done[band], bst) != cudaSuccess ||
                cudaStreamWaitEvent(s->copy_out_stream, s->ev_band_done[band], 0) != cudaSuccess ||
                cudaMemcpyAsync((char *)y_host + off, (const char *)y + off, (size_t)nr * row_bytes, cudaMemcpyDeviceToHost,
                                s->copy_out_stream) != cudaSuccess)
                return fail("queueing the D2H copy of band %d failed", band);
        }
    }
    if (piped) {  // every copy stream rejoins the caller's stream (the copy-in stream through the lanes that waited on it)
        if (cudaEventRecord(s->ev_copy_join, s->copy_out_stream) != cudaSuccess ||
            cudaStreamWaitEvent(st, s->ev_copy_join, 0) != cudaSuccess)
            return fail("joining the copy streams failed");
    }
    if (two_lanes) {  // the caller's stream continues only when the second lane is done
        if (cudaEventRecord(s->ev_join, s->lane_stream) != cudaSuccess ||
            cudaStreamWaitEvent(st, s->ev_join, 0) != cudaSuccess)
            return fail("joining the second lane failed");
    }
    s->launches_per_forward = launches;
    return 0;
}

int alloc_scratch(Stack *s, Stack::Scratch *w) {
    const size_t e = esize(s->dtype);
    const int wide = s->hidden > s->d ? s->hidden : s->d;
    if (dev_alloc(s, (void **)&w->a8, (size_t)s->band_rows * wide)) return 1;
    if (dev_alloc(s, (void **)&w->a8_scales, (size_t)s->band_rows * sizeof(float))) return 1;
    if (dev_alloc(s, (void **)&w->a8_alt, (size_t)s->band_rows * wide)) return 1;
    if (dev_alloc(s, (void **)&w->a8_alt_scales, (size_t)s->band_rows * sizeof(float))) return 1;
    if (dev_alloc(s, &w->qkv, (size_t)s->band_rows * s->n_qkv * e)) return 1;
    if (dev_alloc(s, (void **)&w->h, (size_t)s->band_rows * s->hidden * sizeof(float))) return 1;
    return 0;
}

}  // namespace

}  // namespace b200

using namespace b200;

extern "C" {

void b200_w8a8_stack_destroy(void *handle);

void *b200_w8a8_stack_create(int d_model, int n_qkv, int d_hidden, int n_layers, int max_rows, int band_rows,
                             int act_dtype, float eps) {
    if (d_model <= 0 || n_qkv < d_model || d_hidden <= 0 || n_layers <= 0 || max_rows <= 0 ||
        (act_dtype != B200_DT_F16 && act_dtype != B200_DT_BF16) || d_model % 128 || d_hidden % 128 || n_qkv % 8) {
        fail("invalid stack configuration d=%d n_qkv=%d hidden=%d layers=%d rows=%d dtype=%d", d_model, n_qkv,
             d_hidden, n_layers, max_rows, act_dtype);
        return nullptr;
    }
    status_slot(true);  // the status word exists before the first (possibly captured) forward
    Stack *s = new Stack();
    s->d = d_model; s->n_qkv = n_qkv; s->hidden = d_hidden; s->n_layers = n_layers; s->max_rows = max_rows;
    s->band_rows = band_rows > 0 && band_rows < max_rows ? band_rows : max_rows;
    s->dtype = act_dtype; s->eps = eps;
    s->fuse_ok = d_model % 256 == 0 && d_model <= 2048 && n_qkv % 32 == 0;
    s->layers.resize((size_t)n_layers);
    cudaGetDevice(&s->device);
    const size_t e = esize(act_dtype);
    bool ok = true;
    for (int i = 0; i < 3 && ok; ++i) ok = !dev_alloc(s, &s->tok[i], (size_t)max_rows * d_model * e);
    ok = ok && !alloc_scratch(s, &s->scratch[0]);
    ok = ok && !dev_alloc(s, &s->host_stage, (size_t)max_rows * d_model * e);
    ok = ok && !dev_alloc(s, &s->host_out, (size_t)max_rows * d_model * e);
    ok = ok && cudaStreamCreateWithFlags(&s->own_stream, cudaStreamNonBlocking) == cudaSuccess;
    if (!ok) {
        b200_w8a8_stack_destroy(s);
        return nullptr;
    }
    return s;
}

void b200_w8a8_stack_destroy(void *handle) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s) return;
    for (auto &kv : s->graphs) cudaGraphExecDestroy(kv.second);
    for (auto &kv : s->host_graphs) cudaGraphExecDestroy(kv.second);
    for (cudaEvent_t e : s->ev_band_in) cudaEventDestroy(e);
    for (cudaEvent_t e : s->ev_band_done) cudaEventDestroy(e);
    if (s->copy_in_stream) cudaStreamDestroy(s->copy_in_stream);
    if (s->copy_out_stream) cudaStreamDestroy(s->copy_out_stream);
    if (s->ev_copy_fork) cudaEventDestroy(s->ev_copy_fork);
    if (s->ev_copy_join) cudaEventDestroy(s->ev_copy_join);
    for (auto &L : s->layers) {
        Weight *ws[5] = {&L.qkv, &L.out, &L.ctrl, &L.up, &L.down};
        for (Weight *w : ws) {
            cudaFree(w->codes);
            cudaFree(w->scales);
        }
        cudaFree(L.g_attn);
        cudaFree(L.g_ctrl);
        cudaFree(L.g_mlp);
    }
    for (int i = 0; i < 3; ++i) cudaFree(s->tok[i]);
    for (auto &w : s->scratch) {
        cudaFree(w.a8);
        cudaFree(w.a8_scales);
        cudaFree(w.a8_alt);
        cudaFree(w.a8_alt_scales);
        cudaFree(w.qkv);
        cudaFree(w.h);
    }
    if (s->lane_stream) cudaStreamDestroy(s->lane_stream);
    if (s->ev_fork) cudaEventDestroy(s->ev_fork);
    if (s->ev_join) cudaEventDestroy(s->ev_join);
    cudaFree(s->host_stage);
    cudaFree(s->host_out);
    if (s->own_stream) cudaStreamDestroy(s->own_stream);
    delete s;
}

int b200_w8a8_stack_set_layer(void *handle, int layer, const float *w_qkv, const float *w_out, const float *w_ctrl,
                              const float *w_up, const float *w_down, const float *g_attn, const float *g_ctrl,
                              const float *g_mlp, int threads) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s || layer < 0 || layer >= s->n_layers || !w_qkv || !w_out || !w_ctrl || !w_up || !w_down || !g_attn ||
        !g_ctrl || !g_mlp)
        return fail("invalid stack_set_layer arguments (layer %d)", layer);
    Layer &L = s->layers[(size_t)layer];
    if (upload_weight(s, &L.qkv, w_qkv, s->n_qkv, s->d, threads)) return 1;
    if (upload_weight(s, &L.out, w_out, s->d, s->d, threads)) return 1;
    if (upload_weight(s, &L.ctrl, w_ctrl, s->d, s->d, threads)) return 1;
    if (upload_weight(s, &L.up, w_up, s->hidden, s->d, threads)) return 1;
    if (upload_weight(s, &L.down, w_down, s->d, s->hidden, threads)) return 1;
    if (upload_vec(s, &L.g_attn, g_attn, s->d)) return 1;
    if (upload_vec(s, &L.g_ctrl, g_ctrl, s->d)) return 1;
    if (upload_vec(s, &L.g_mlp, g_mlp, s->d)) return 1;
    L.loaded = true;
    return 0;
}

// Copies one layer record of a packed-weight file (host memory, file order) to the device.
static int upload_record(Stack *s, Layer &L, const uint8_t *rec) {
    Weight *ws[5] = {&L.qkv, &L.out, &L.ctrl, &L.up, &L.down};
    const int ns[5] = {s->n_qkv, s->d, s->d, s->hidden, s->d};
    const int ks[5] = {s->d, s->d, s->d, s->d, s->hidden};
    cudaError_t e = cudaSuccess;
    for (int i = 0; i < 5 && e == cudaSuccess; ++i) {
        const size_t cb = packed_weight_bytes(ns[i], ks[i], B200_W_SLAB128), sb = (size_t)ns[i] * sizeof(float);
        if (!ws[i]->codes) {
            if (dev_alloc(s, (void **)&ws[i]->codes, cb)) return 1;
            if (dev_alloc(s, (void **)&ws[i]->scales, sb)) return 1;
        }
        ws[i]->n = ns[i];
        ws[i]->k = ks[i];
        e = cudaMemcpy(ws[i]->codes, rec, cb, cudaMemcpyHostToDevice);
        if (e == cudaSuccess) e = cudaMemcpy(ws[i]->scales, rec + cb, sb, cudaMemcpyHostToDevice);
        rec += cb + sb;
    }
    float **gs[3] = {&L.g_attn, &L.g_ctrl, &L.g_mlp};
    const size_t gb = (size_t)s->d * sizeof(float);
    for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
        if (!*gs[i] && dev_alloc(s, (void **)gs[i], gb)) return 1;
        e = cudaMemcpy(*gs[i], rec, gb, cudaMemcpyHostToDevice);
        rec += gb;
    }
    if (e != cudaSuccess) return fail("CUDA error while copying packed weights: %s", cudaGetErrorString(e));
    L.loaded = true;
    return 0;
}

int b200_w8a8_stack_load_weights(void *handle, const char *path) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s || !path) return fail("invalid stack_load_weights arguments");
    int d = 0, nq = 0, hid = 0, nl = 0;
    if (weight_file_info(path, &d, &nq, &hid, &nl, 1)) return 1;
    if (d != s->d || nq != s->n_qkv || hid != s->hidden || nl != s->n_layers)
        return fail("%s holds d=%d n_qkv=%d hidden=%d layers=%d, the stack is d=%d n_qkv=%d hidden=%d layers=%d", path,
                    d, nq, hid, nl, s->d, s->n_qkv, s->hidden, s->n_layers);
    std::vector<uint8_t> rec(weight_file_layer_bytes(d, nq, hid));
    for (int l = 0; l < nl; ++l) {
        if (weight_file_read_layer(path, l, d, nq, hid, rec.data())) return 1;
        if (upload_record(s, s->layers[(size_t)l], rec.data())) return 1;
    }
    return 0;
}

int b200_w8a8_stack_save_weights(void *handle, const char *path) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s || !path) return fail("invalid stack_save_weights arguments");
    for (const Layer &L : s->layers)
        if (!L.loaded) return fail("stack_save_weights called before every layer was loaded");
    WeightFileWriter *w = weight_file_create(path, s->d, s->n_qkv, s->hidden, s->n_layers);
    if (!w) return 1;
    int rc = 0;
    for (const Layer &L : s->layers) {
        const Weight *ws[5] = {&L.qkv, &L.out, &L.ctrl, &L.up, &L.down};
        std::vector<int8_t> codes[5];
        std::vector<float> scales[5], gammas[3];
        const int8_t *cp[5];
        const float *sp[5], *gp[3];
        cudaError_t e = cudaSuccess;
        for (int i = 0; i < 5 && e == cudaSuccess; ++i) {
            codes[i].resize(packed_weight_bytes(ws[i]->n, ws[i]->k, B200_W_SLAB128));
            scales[i].resize((size_t)ws[i]->n);
            e = cudaMemcpy(codes[i].data(), ws[i]->codes, codes[i].size(), cudaMemcpyDeviceToHost);
            if (e == cudaSuccess)
                e = cudaMemcpy(scales[i].data(), ws[i]->scales, scales[i].size() * sizeof(float), cudaMemcpyDeviceToHost);
            cp[i] = codes[i].data();
            sp[i] = scales[i].data();
        }
        const float *gd[3] = {L.g_attn, L.g_ctrl, L.g_mlp};
        for (int i = 0; i < 3 && e == cudaSuccess; ++i) {
            gammas[i].resize((size_t)s->d);
            e = cudaMemcpy(gammas[i].data(), gd[i], (size_t)s->d * sizeof(float), cudaMemcpyDeviceToHost);
            gp[i] = gammas[i].data();
        }
        if (e != cudaSuccess) rc = fail("CUDA error while reading back packed weights: %s", cudaGetErrorString(e));
        if (!rc) rc = weight_file_add_packed(w, cp, sp, gp);
        if (rc) break;
    }
    const int rc_close = weight_file_close(w);
    return rc ? rc : rc_close;
}

int b200_w8a8_stack_set_lanes(void *handle, int lanes) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s || lanes < 1 || lanes > 2) return fail("invalid stack_set_lanes (1 or 2 lanes)");
    if (lanes == 2 && !s->lane_stream) {
        if (alloc_scratch(s, &s->scratch[1])) return 1;
        if (cudaStreamCreateWithFlags(&s->lane_stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->ev_fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&s->ev_join, cudaEventDisableTiming) != cudaSuccess)
            return fail("creating the second lane's stream failed");
    }
    if (lanes != s->lanes) {
        for (auto &kv : s->graphs) cudaGraphExecDestroy(kv.second);
        s->graphs.clear();
        for (auto &kv : s->host_graphs) cudaGraphExecDestroy(kv.second);
        s->host_graphs.clear();
        s->lanes = lanes;
    }
    return 0;
}

int b200_w8a8_stack_set_fusion(void *handle, int on) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s) return fail("invalid stack_set_fusion");
    if ((on != 0) != (s->fusion != 0)) {
        for (auto &kv : s->graphs) cudaGraphExecDestroy(kv.second);
        s->graphs.clear();
        for (auto &kv : s->host_graphs) cudaGraphExecDestroy(kv.second);
        s->host_graphs.clear();
        s->fusion = on != 0;
    }
    return 0;
}

int b200_w8a8_stack_set_act_dtype(void *handle, int act_dtype) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (!s || (act_dtype != B200_DT_F16 && act_dtype != B200_DT_BF16)) return fail("invalid stack_set_act_dtype");
    if (act_dtype != s->dtype) {
        for (auto &kv : s->graphs) cudaGraphExecDestroy(kv.second);  // captured launches bake the type in
        s->graphs.clear();
        for (auto &kv : s->host_graphs) cudaGraphExecDestroy(kv.second);
        s->host_graphs.clear();
        s->dtype = act_dtype;
    }
    return 0;
}

size_t b200_w8a8_stack_device_bytes(void *handle) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    return s ? s->device_bytes : 0;
}

long long b200_w8a8_stack_launches_per_forward(void *handle) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    return s ? s->launches_per_forward : 0;
}

int b200_w8a8_stack_forward(void *handle, const void *x_dev, void *y_dev, int rows, int steps, int use_graph,
                            void *stream) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (status_check_entry()) return 1;
    if (!s || !x_dev || !y_dev || rows <= 0 || rows > s->max_rows || steps <= 0)
        return fail("invalid stack_forward arguments rows=%d steps=%d", rows, steps);
    for (const Layer &L : s->layers)
        if (!L.loaded) return fail("stack_forward called before every layer was loaded");
    cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);  // NULL = the legacy default stream
    if (!use_graph) return enqueue(s, x_dev, y_dev, rows, steps, st);

    auto key = std::make_tuple(x_dev, y_dev, rows, steps);
    auto it = s->graphs.find(key);
    if (it == s->graphs.end()) {
        if (!stream || st == cudaStreamLegacy || stream == B200_STREAM_PER_THREAD)
            return fail("graph replay needs a capturable stream (not a default stream)");
        cudaGraph_t graph = nullptr;
        cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
        if (e != cudaSuccess) return fail("cudaStreamBeginCapture: %s", cudaGetErrorString(e));
        const int rc = enqueue(s, x_dev, y_dev, rows, steps, st);
        e = cudaStreamEndCapture(st, &graph);
        if (rc || e != cudaSuccess || !graph) {
            if (graph) cudaGraphDestroy(graph);
            return rc ? 1 : fail("cudaStreamEndCapture: %s", cudaGetErrorString(e));
        }
        cudaGraphExec_t exec = nullptr;
        e = cudaGraphInstantiate(&exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess) return fail("cudaGraphInstantiate: %s", cudaGetErrorString(e));
        it = s->graphs.emplace(key, exec).first;
    }
    cudaError_t e = cudaGraphLaunch(it->second, st);
    if (e != cudaSuccess) return fail("cudaGraphLaunch: %s", cudaGetErrorString(e));
    return 0;
}

int b200_w8a8_stack_forward_host(void *handle, const void *x_host, void *y_host, int rows, int steps, int use_graph) {
    Stack *s = reinterpret_cast<Stack *>(handle);
    if (status_check_entry()) return 1;
    if (!s || !x_host || !y_host || rows <= 0 || rows > s->max_rows || steps <= 0)
        return fail("invalid stack_forward_host arguments rows=%d steps=%d", rows, steps);
    for (const Layer &L : s->layers)
        if (!L.loaded) return fail("stack_forward_host called before every layer was loaded");
    cudaStream_t st = s->own_stream;
    cudaError_t e = cudaSuccess;
    if (!use_graph) {
        if (enqueue(s, s->host_stage, s->host_out, rows, steps, st, x_host, y_host)) return 1;
    } else {
        // copies and kernels of all bands as one graph: the host pointers are part of the key
        auto key = std::make_tuple(x_host, y_host, rows, steps);
        auto it = s->host_graphs.find(key);
        if (it == s->host_graphs.end()) {
            const int n_bands = (rows + s->band_rows - 1) / s->band_rows;
            if (ensure_copy_pipeline(s, n_bands)) return 1;  // nothing is created while the capture runs
            cudaGraph_t graph = nullptr;
            e = cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal);
            if (e != cudaSuccess) return fail("cudaStreamBeginCapture: %s", cudaGetErrorString(e));
            const int rc = enqueue(s, s->host_stage, s->host_out, rows, steps, st, x_host, y_host);
            e = cudaStreamEndCapture(st, &graph);
            if (rc || e != cudaSuccess || !graph) {
                if (graph) cudaGraphDestroy(graph);
                return rc ? 1 : fail("cudaStreamEndCapture: %s", cudaGetErrorString(e));
            }
            cudaGraphExec_t exec = nullptr;
            e = cudaGraphInstantiate(&exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e != cudaSuccess) return fail("cudaGraphInstantiate: %s", cudaGetErrorString(e));
            it = s->host_graphs.emplace(key, exec).first;
        }
        e = cudaGraphLaunch(it->second, st);
        if (e != cudaSuccess) return fail("cudaGraphLaunch: %s", cudaGetErrorString(e));
    }
    e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail("synchronizing the host entry point: %s", cudaGetErrorString(e));
    return 0;
}

}  // extern "C"
