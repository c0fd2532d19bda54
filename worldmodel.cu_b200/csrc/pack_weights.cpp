// Host-side weight preparation: per-output-channel symmetric int8 quantization of fp32
// weights and placement into the layout the GEMM streams.
//
// It replaces the reference's single-threaded quantize-then-upload helper
// (src/world_cuda.cu:153-222).  Rows are independent, so they are split over host threads.
// The rounding rule is the activation quantizer's (scale = amax / 127 with IEEE division,
// code = rne(w / scale) clamped to +-127, an all-zero row gets scale 1), and non-finite
// weights are rejected like the reference does.
#include <math.h>
#include <string.h>

#include <atomic>
#include <thread>
#include <vector>

#include "w8a8_internal.h"

namespace b200 {

size_t packed_weight_bytes(int n, int k, int layout) {
    if (n <= 0 || k <= 0) return 0;
    if (layout == B200_W_SLAB128 && (k % 128) != 0) return 0;
    return (size_t)n * (size_t)k;
}

int pack_weight_host(const float *w, int n, int k, int layout, int8_t *packed, float *scales, int threads) {
    if (!w || !packed || !scales || n <= 0 || k <= 0) return fail("invalid pack_weight arguments N=%d K=%d", n, k);
    if (layout != B200_W_ROW_MAJOR && layout != B200_W_SLAB128) return fail("unknown weight layout %d", layout);
    if (layout == B200_W_SLAB128 && (k % 128) != 0)
        return fail("the slab weight layout needs K %% 128 == 0, got K=%d", k);
    if (threads <= 0) threads = (int)std::thread::hardware_concurrency();
    if (threads <= 0) threads = 1;
    if (threads > n) threads = n;

    std::atomic<int> bad_row(-1), bad_col(-1);
    auto work = [&](int r0, int r1) {
        std::vector<int8_t> codes((size_t)k);
        for (int row = r0; row < r1; ++row) {
            const float *src = w + (size_t)row * k;
            float amax = 0.0f;
            for (int c = 0; c < k; ++c) {
                if (!isfinite(src[c])) {
                    int expect = -1;
                    if (bad_row.compare_exchange_strong(expect, row)) bad_col.store(c);
                    return;
                }
                amax = fmaxf(amax, fabsf(src[c]));
            }
            const float scale = amax > 0.0f ? amax / 127.0f : 1.0f;
            scales[row] = scale;
            for (int c = 0; c < k; ++c) {
                int v = (int)nearbyintf(src[c] / scale);  // ties to even in the default rounding mode
                v = v < -127 ? -127 : (v > 127 ? 127 : v);
                codes[c] = (int8_t)v;
            }
            if (layout == B200_W_ROW_MAJOR) {
                memcpy(packed + (size_t)row * k, codes.data(), (size_t)k);
            } else {
                for (int slab = 0; slab < k / 128; ++slab)
                    memcpy(packed + ((size_t)slab * n + row) * 128, codes.data() + (size_t)slab * 128, 128);
            }
        }
    };
    std::vector<std::thread> pool;
    const int per = (n + threads - 1) / threads;
    for (int t = 0; t < threads; ++t) {
        int r0 = t * per, r1 = r0 + per > n ? n : r0 + per;
        if (r0 >= r1) break;
        pool.emplace_back(work, r0, r1);
    }
    for (auto &th : pool) th.join();
    if (bad_row.load() >= 0)
        return fail("weight matrix [%d,%d] holds a value that is not finite at row %d, column %d", n, k, bad_row.load(), bad_col.load());
    return 0;
}

// The 128 x 128 blockwise rule (docs/cuda_w8a8_optimization.md:319-321 of the reference describes it):
// one scale per block, scale = max(amax, 1e-8) / 128, codes rne(w / scale) saturated to [-128, 127];
// scales[ceil(n / 128)][k / 128].  Block rows are independent and go to separate host threads.
int pack_weight_blocks128_host(const float *w, int n, int k, int layout, int8_t *packed, float *scales, int threads) {
    if (!w || !packed || !scales || n <= 0 || k <= 0) return fail("invalid pack_weight_blocks128 arguments N=%d K=%d", n, k);
    if (layout != B200_W_ROW_MAJOR && layout != B200_W_SLAB128) return fail("unknown weight layout %d", layout);
    if ((k % 128) != 0) return fail("blockwise weights need K %% 128 == 0, got K=%d", k);
    const int nb = (n + 127) / 128, kbs = k / 128;
    if (threads <= 0) threads = (int)std::thread::hardware_concurrency();
    if (threads <= 0) threads = 1;
    if (threads > nb) threads = nb;
    std::atomic<int> bad_row(-1), bad_col(-1);
    std::atomic<int> next(0);
    auto work = [&]() {
        for (int b = next.fetch_add(1); b < nb; b = next.fetch_add(1)) {
            const int r0 = b * 128, r1 = r0 + 128 > n ? n : r0 + 128;
            for (int kb = 0; kb < kbs; ++kb) {
                float amax = 0.0f;
                for (int row = r0; row < r1; ++row) {
                    const float *src = w + (size_t)row * k + (size_t)kb * 128;
                    for (int c = 0; c < 128; ++c) {
                        if (!isfinite(src[c])) {
                            int expect = -1;
                            if (bad_row.compare_exchange_strong(expect, row)) bad_col.store(kb * 128 + c);
                            return;
                        }
                        amax = fmaxf(amax, fabsf(src[c]));
                    }
                }
                const float scale = fmaxf(amax, 1e-8f) / 128.0f;
                scales[(size_t)b * kbs + kb] = scale;
                for (int row = r0; row < r1; ++row) {
                    const float *src = w + (size_t)row * k + (size_t)kb * 128;
                    int8_t *dst = layout == B200_W_ROW_MAJOR ? packed + (size_t)row * k + (size_t)kb * 128
                                                             : packed + ((size_t)kb * n + row) * 128;
                    for (int c = 0; c < 128; ++c) {
                        int v = (int)nearbyintf(src[c] / scale);  // ties to even in the default rounding mode
                        dst[c] = (int8_t)(v < -128 ? -128 : (v > 127 ? 127 : v));
                    }
                }
            }
        }
    };
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t) pool.emplace_back(work);
    for (auto &th : pool) th.join();
    if (bad_row.load() >= 0)
        return fail("weight matrix [%d,%d] holds a value that is not finite at row %d, column %d", n, k, bad_row.load(), bad_col.load());
    return 0;
}

}  // namespace b200
