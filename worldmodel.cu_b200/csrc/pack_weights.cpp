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

}  // namespace b200
