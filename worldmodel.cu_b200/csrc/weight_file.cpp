// Offline packed-weight file of the linear stack: the int8 codes (already in the slab
// layout the GEMM's tensor maps read) and the fp32 per-channel scales of every layer,
// written once on any host and copied to the device at start-up without touching the
// fp32 checkpoint.  The reference re-quantizes the fp32 weights on every start
// (copy_f32_to_i8_per_output_device, src/world_cuda.cu:153-222) and lists the offline
// export as the next step of its roadmap (docs/cuda_w8a8_optimization.md:357).
//
// Layout (little endian):
//   FileHeader (64 bytes)
//   per layer, in order: qkv, out, ctrl, up, down  -> codes[packed bytes], scales[n] fp32
//                        g_attn[d], g_ctrl[d], g_mlp[d] fp32
// `checksum` is FNV-1a (64 bit) over everything after the header.  Host-only code: no
// CUDA call in this file, so the writer runs where there is no GPU.
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "w8a8_internal.h"

namespace b200 {

namespace {

const char kMagic[8] = {'B', '2', 'W', '8', 'A', '8', 'W', 'F'};
const uint32_t kVersion = 1;

struct FileHeader {
    char magic[8];
    uint32_t version;
    uint32_t layout;
    uint32_t d, n_qkv, hidden, n_layers;
    uint64_t payload_bytes;
    uint64_t checksum;
    uint8_t reserved[16];
};
static_assert(sizeof(FileHeader) == 64, "the header is 64 bytes on disk");

uint64_t fnv1a(uint64_t h, const void *data, size_t n) {
    const uint8_t *p = static_cast<const uint8_t *>(data);
    for (size_t i = 0; i < n; ++i) h = (h ^ p[i]) * 1099511628211ull;
    return h;
}
const uint64_t kFnvSeed = 1469598103934665603ull;

bool dims_ok(int d, int n_qkv, int hidden, int n_layers) {
    return d > 0 && n_qkv >= d && hidden > 0 && n_layers > 0 && d % 128 == 0 && hidden % 128 == 0 && n_qkv % 8 == 0;
}

}  // namespace

size_t weight_file_layer_bytes(int d, int n_qkv, int hidden) {
    const int ns[5] = {n_qkv, d, d, hidden, d};
    const int ks[5] = {d, d, d, d, hidden};
    size_t b = 0;
    for (int i = 0; i < 5; ++i) b += packed_weight_bytes(ns[i], ks[i], B200_W_SLAB128) + (size_t)ns[i] * sizeof(float);
    return b + 3 * (size_t)d * sizeof(float);
}

struct WeightFileWriter {
    FILE *f = nullptr;
    int d = 0, n_qkv = 0, hidden = 0, n_layers = 0, next_layer = 0;
    uint64_t hash = kFnvSeed, bytes = 0;
    bool failed = false;

    void put(const void *p, size_t n) {
        if (failed) return;
        if (fwrite(p, 1, n, f) != n) failed = true;
        hash = fnv1a(hash, p, n);
        bytes += n;
    }
};

WeightFileWriter *weight_file_create(const char *path, int d, int n_qkv, int hidden, int n_layers) {
    if (!path || !dims_ok(d, n_qkv, hidden, n_layers)) {
        fail("invalid weight file configuration d=%d n_qkv=%d hidden=%d layers=%d", d, n_qkv, hidden, n_layers);
        return nullptr;
    }
    FILE *f = fopen(path, "wb");
    if (!f) {
        fail("cannot open %s for writing", path);
        return nullptr;
    }
    FileHeader h{};  // rewritten with the checksum when the file is closed
    if (fwrite(&h, sizeof(h), 1, f) != 1) {
        fclose(f);
        fail("cannot write to %s", path);
        return nullptr;
    }
    WeightFileWriter *w = new WeightFileWriter();
    w->f = f; w->d = d; w->n_qkv = n_qkv; w->hidden = hidden; w->n_layers = n_layers;
    return w;
}

int weight_file_add_packed(WeightFileWriter *w, const int8_t *const codes[5], const float *const scales[5],
                           const float *const gammas[3]) {
    if (!w || w->next_layer >= w->n_layers) return fail("weight file: more layers added than declared");
    const int ns[5] = {w->n_qkv, w->d, w->d, w->hidden, w->d};
    const int ks[5] = {w->d, w->d, w->d, w->d, w->hidden};
    for (int i = 0; i < 5; ++i) {
        w->put(codes[i], packed_weight_bytes(ns[i], ks[i], B200_W_SLAB128));
        w->put(scales[i], (size_t)ns[i] * sizeof(float));
    }
    for (int i = 0; i < 3; ++i) w->put(gammas[i], (size_t)w->d * sizeof(float));
    ++w->next_layer;
    return w->failed ? fail("weight file: short write") : 0;
}

int weight_file_add_layer(WeightFileWriter *w, const float *const weights[5], const float *const gammas[3],
                          int threads) {
    if (!w) return fail("weight file: null writer");
    const int ns[5] = {w->n_qkv, w->d, w->d, w->hidden, w->d};
    const int ks[5] = {w->d, w->d, w->d, w->d, w->hidden};
    std::vector<int8_t> codes[5];
    std::vector<float> scales[5];
    const int8_t *cp[5];
    const float *sp[5];
    for (int i = 0; i < 5; ++i) {
        if (!weights[i]) return fail("weight file: null weight %d", i);
        codes[i].resize(packed_weight_bytes(ns[i], ks[i], B200_W_SLAB128));
        scales[i].resize((size_t)ns[i]);
        if (pack_weight_host(weights[i], ns[i], ks[i], B200_W_SLAB128, codes[i].data(), scales[i].data(), threads))
            return 1;
        cp[i] = codes[i].data();
        sp[i] = scales[i].data();
    }
    for (int i = 0; i < 3; ++i)
        if (!gammas[i]) return fail("weight file: null norm vector %d", i);
    return weight_file_add_packed(w, cp, sp, gammas);
}

int weight_file_close(WeightFileWriter *w) {
    if (!w) return fail("weight file: null writer");
    int rc = 0;
    if (w->next_layer != w->n_layers)
        rc = fail("weight file closed after %d of %d layers", w->next_layer, w->n_layers);
    FileHeader h{};
    memcpy(h.magic, kMagic, 8);
    h.version = kVersion; h.layout = B200_W_SLAB128;
    h.d = (uint32_t)w->d; h.n_qkv = (uint32_t)w->n_qkv; h.hidden = (uint32_t)w->hidden;
    h.n_layers = (uint32_t)w->n_layers;
    h.payload_bytes = w->bytes; h.checksum = w->hash;
    if (!rc && (w->failed || fseek(w->f, 0, SEEK_SET) != 0 || fwrite(&h, sizeof(h), 1, w->f) != 1))
        rc = fail("weight file: writing the header failed");
    if (fclose(w->f) != 0 && !rc) rc = fail("weight file: close failed");
    delete w;
    return rc;
}

// Reads and validates the header; with `verify` also re-hashes the payload.
int weight_file_info(const char *path, int *d, int *n_qkv, int *hidden, int *n_layers, int verify) {
    if (!path) return fail("weight file: null path");
    FILE *f = fopen(path, "rb");
    if (!f) return fail("cannot open %s", path);
    FileHeader h{};
    int rc = 0;
    if (fread(&h, sizeof(h), 1, f) != 1 || memcmp(h.magic, kMagic, 8) != 0)
        rc = fail("%s is not a packed W8A8 weight file", path);
    else if (h.version != kVersion || h.layout != (uint32_t)B200_W_SLAB128)
        rc = fail("%s: unsupported version %u / layout %u", path, h.version, h.layout);
    else if (h.d > (1u << 20) || h.n_qkv > (1u << 22) || h.hidden > (1u << 22) || h.n_layers > (1u << 16) ||
             !dims_ok((int)h.d, (int)h.n_qkv, (int)h.hidden, (int)h.n_layers))
        rc = fail("%s: invalid dimensions in the header", path);
    else if (h.payload_bytes != (uint64_t)weight_file_layer_bytes((int)h.d, (int)h.n_qkv, (int)h.hidden) * h.n_layers)
        rc = fail("%s: payload size does not match the dimensions", path);
    if (!rc && verify) {
        std::vector<uint8_t> buf(1 << 22);
        uint64_t hash = kFnvSeed, left = h.payload_bytes;
        while (left) {
            const size_t want = left < buf.size() ? (size_t)left : buf.size();
            if (fread(buf.data(), 1, want, f) != want) {
                rc = fail("%s is truncated", path);
                break;
            }
            hash = fnv1a(hash, buf.data(), want);
            left -= want;
        }
        if (!rc && hash != h.checksum) rc = fail("%s: checksum mismatch", path);
        if (!rc && fgetc(f) != EOF) rc = fail("%s: trailing bytes after the payload", path);
    }
    fclose(f);
    if (!rc) {
        if (d) *d = (int)h.d;
        if (n_qkv) *n_qkv = (int)h.n_qkv;
        if (hidden) *hidden = (int)h.hidden;
        if (n_layers) *n_layers = (int)h.n_layers;
    }
    return rc;
}

// Reads layer `layer` (whole record) into `dst`, which holds weight_file_layer_bytes().
int weight_file_read_layer(const char *path, int layer, int d, int n_qkv, int hidden, void *dst) {
    FILE *f = fopen(path, "rb");
    if (!f) return fail("cannot open %s", path);
    const size_t lb = weight_file_layer_bytes(d, n_qkv, hidden);
    int rc = 0;
    if (fseek(f, (long)(sizeof(FileHeader) + lb * (size_t)layer), SEEK_SET) != 0 || fread(dst, 1, lb, f) != lb)
        rc = fail("%s: reading layer %d failed", path, layer);
    fclose(f);
    return rc;
}

}  // namespace b200

using namespace b200;

extern "C" {

void *b200_w8a8_weight_file_create(const char *path, int d_model, int n_qkv, int d_hidden, int n_layers) {
    return weight_file_create(path, d_model, n_qkv, d_hidden, n_layers);
}

int b200_w8a8_weight_file_add_layer(void *writer, const float *w_qkv, const float *w_out, const float *w_ctrl,
                                    const float *w_up, const float *w_down, const float *g_attn,
                                    const float *g_ctrl, const float *g_mlp, int threads) {
    const float *ws[5] = {w_qkv, w_out, w_ctrl, w_up, w_down};
    const float *gs[3] = {g_attn, g_ctrl, g_mlp};
    return weight_file_add_layer(static_cast<WeightFileWriter *>(writer), ws, gs, threads);
}

int b200_w8a8_weight_file_close(void *writer) { return weight_file_close(static_cast<WeightFileWriter *>(writer)); }

int b200_w8a8_weight_file_info(const char *path, int *d_model, int *n_qkv, int *d_hidden, int *n_layers, int verify) {
    return weight_file_info(path, d_model, n_qkv, d_hidden, n_layers, verify);
}

}  // extern "C"
