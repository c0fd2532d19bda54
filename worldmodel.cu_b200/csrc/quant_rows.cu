// Per-token activation quantizers: plain absmax -> A8, fused (Ada)RMSNorm -> A8, and
// dequant -> bias -> activation -> A8 of an int32 accumulator.
//
// They replace the reference's one-CTA-per-row, scalar, three-pass kernels
// (src/world_cuda_ops.cu:94-125, 129-182, 187-227).  Here a row is owned by a group of
// G threads (one warp, or the whole 256-thread CTA), is read from global memory exactly
// once with 16/32-byte vector loads, lives in registers across the reductions, and is
// written back as packed 8-byte code vectors.  Reductions are warp shuffles (plus one
// shared-memory hop when G spans several warps).  All of these kernels are bound by HBM
// traffic: bytes in + 1 byte per element out.
#include "common.cuh"
#include "w8a8_internal.h"

namespace b200 {

namespace {

constexpr int kThreads = 256;
constexpr int kMaxVec = 8;  // 8-element vectors held per thread

enum Mode { MODE_PLAIN = 0, MODE_RMS = 1, MODE_DEQ_ACT = 2 };

struct QuantArgs {
    const void *x;          // input rows (fp32 / fp16 / bf16 / int32 accumulators)
    long long ldx;          // input row stride in elements
    int8_t *q;              // output codes
    long long ldq;          // output row stride in elements
    float *scales;          // output per-row scales
    int rows, cols;
    // MODE_RMS
    const float *vec_scale;  // gamma or mod_scale, nullable
    const float *vec_bias;   // nullable
    int scale_is_mod;        // 1: multiply by (1 + vec_scale[col])
    float eps;
    double inv_cols;         // 1 / cols when that is exact (cols a power of two), else 0: divide
    // MODE_DEQ_ACT
    const float *in_row_scales;
    const float *col_scales;
    int act;
};

template <typename T>
struct Load8;
template <>
struct Load8<float> {
    static __device__ __forceinline__ void run(const void *p, float (&v)[8]) {
        const float4 *s = reinterpret_cast<const float4 *>(p);
        float4 a = s[0], b = s[1];
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ float one(const void *p, long long i) {
        return reinterpret_cast<const float *>(p)[i];
    }
};
template <>
struct Load8<int32_t> {
    static __device__ __forceinline__ void run(const void *p, float (&v)[8]) {
        const int4 *s = reinterpret_cast<const int4 *>(p);
        int4 a = s[0], b = s[1];
        v[0] = (float)a.x; v[1] = (float)a.y; v[2] = (float)a.z; v[3] = (float)a.w;
        v[4] = (float)b.x; v[5] = (float)b.y; v[6] = (float)b.z; v[7] = (float)b.w;
    }
    static __device__ __forceinline__ float one(const void *p, long long i) {
        return (float)reinterpret_cast<const int32_t *>(p)[i];
    }
};
template <>
struct Load8<__half> {
    static __device__ __forceinline__ void run(const void *p, float (&v)[8]) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __half22float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ float one(const void *p, long long i) {
        return __half2float(reinterpret_cast<const __half *>(p)[i]);
    }
};
template <>
struct Load8<__nv_bfloat16> {
    static __device__ __forceinline__ void run(const void *p, float (&v)[8]) {
        uint4 raw = *reinterpret_cast<const uint4 *>(p);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ float one(const void *p, long long i) {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    }
};

__device__ __forceinline__ void load8f(const float *p, float (&v)[8]) { Load8<float>::run(p, v); }

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Reduction over the G threads that own one row.  For G == 32 it is a pure shuffle; for wider
// groups every warp of the CTA posts its partial to shared memory and each group combines its
// own G/32 entries (the CTA-wide barriers are shared by all row groups of the CTA).
template <int G>
__device__ __forceinline__ float group_max(float v, float *red) {
    v = warp_max(v);
    if (G == 32) return v;
    __syncthreads();  // protect `red` from the previous use
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    const int w0 = (threadIdx.x / G) * (G / 32);
    float r = red[w0];
#pragma unroll
    for (int i = 1; i < G / 32; ++i) r = fmaxf(r, red[w0 + i]);
    return r;
}
template <int G>
__device__ __forceinline__ double group_sum(double v, double *red) {
    v = warp_sum(v);
    if (G == 32) return v;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    const int w0 = (threadIdx.x / G) * (G / 32);
    double r = red[w0];
#pragma unroll
    for (int i = 1; i < G / 32; ++i) r += red[w0 + i];
    return r;
}

// fp32(1 / sqrt(ss / cols + eps)) from the fp64 sum of squares.  The reciprocal square root is
// the fp64 intrinsic (a seed plus Newton steps, within an ulp of fp64), a quarter of the
// instructions of a division and a square root; after rounding to fp32 it differs from the
// correctly rounded value only when that lies within 2^-53 of an fp32 rounding boundary, the
// same order as the summation-order effect on ss itself.
__device__ __forceinline__ float inv_rms_of(double ss, const QuantArgs &a) {
    const double mean = a.inv_cols != 0.0 ? ss * a.inv_cols : ss / (double)a.cols;
    return (float)rsqrt(mean + (double)a.eps);
}

// The transform each mode applies to a loaded vector of 8 elements at column `col`.
template <int MODE>
__device__ __forceinline__ void transform8(float (&v)[8], int col, const QuantArgs &a, float row_factor) {
    if (MODE == MODE_RMS) {
        float s[8], b[8];
        if (a.vec_scale) load8f(a.vec_scale + col, s);
        if (a.vec_bias) load8f(a.vec_bias + col, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float t = __fmul_rn(v[i], row_factor);
            if (a.vec_scale) t = __fmul_rn(t, a.scale_is_mod ? __fadd_rn(1.0f, s[i]) : s[i]);
            if (a.vec_bias) t = __fadd_rn(t, b[i]);
            v[i] = t;
        }
    } else if (MODE == MODE_DEQ_ACT) {
        float s[8], b[8];
        load8f(a.col_scales + col, s);
        if (a.vec_bias) load8f(a.vec_bias + col, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float t = __fmul_rn(__fmul_rn(v[i], row_factor), s[i]);
            if (a.vec_bias) t = __fadd_rn(t, b[i]);
            v[i] = apply_act_rt(t, a.act);
        }
    }
}

// Fast path: cols % 8 == 0, 16-byte aligned rows, cols <= G * 8 * NV.  NV (vectors of 8
// elements held per thread) is a template argument so that narrow rows do not pay the
// register footprint of wide ones: occupancy is what hides the load latency here.
template <typename T, int MODE, int G, int NV>
__global__ void __launch_bounds__(kThreads) quant_rows_vec_kernel(QuantArgs a) {
    __shared__ float red_f[kThreads / 32];
    __shared__ double red_d[kThreads / 32];
    pdl_trigger();
    pdl_wait();
    constexpr int kRowsPerCta = kThreads / G;
    const int gid = threadIdx.x / G;
    const int gl = threadIdx.x % G;
    const int row = blockIdx.x * kRowsPerCta + gid;
    const bool live = row < a.rows;
    const int nvec = a.cols >> 3;

    const T *xrow = reinterpret_cast<const T *>(a.x) + (long long)row * a.ldx;
    float v[NV][8];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int vi = gl + j * G;
        if (live && vi < nvec) {
            Load8<T>::run(xrow + 8 * vi, v[j]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = 0.0f;
        }
    }

    float row_factor = 1.0f;
    if (MODE == MODE_RMS) {
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                double d = (double)v[j][i];
                ss = fma(d, d, ss);
            }
        }
        ss = group_sum<G>(ss, red_d);
        // the fp64 divide and square root run on one lane per warp; the fp32 result is broadcast
        float f = 0.0f;
        if ((threadIdx.x & 31) == 0) f = inv_rms_of(ss, a);
        row_factor = __shfl_sync(0xffffffffu, f, 0);
    } else if (MODE == MODE_DEQ_ACT) {
        // read before any store: the output scale vector may alias this one
        row_factor = live ? a.in_row_scales[row] : 0.0f;
    }

    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int vi = gl + j * G;
        if (live && vi < nvec) {
            transform8<MODE>(v[j], 8 * vi, a, row_factor);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[j][i]));
        }
    }
    amax = group_max<G>(amax, red_f);
    const RowScale scale = make_row_scale(amax);
    if (live && gl == 0) a.scales[row] = scale.scale;

    int8_t *qrow = a.q + (long long)row * a.ldq;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        int vi = gl + j * G;
        if (live && vi < nvec) {
            const uint32_t lo = pack_biased4(quantize_biased(v[j][0], scale), quantize_biased(v[j][1], scale),
                                             quantize_biased(v[j][2], scale), quantize_biased(v[j][3], scale));
            const uint32_t hi = pack_biased4(quantize_biased(v[j][4], scale), quantize_biased(v[j][5], scale),
                                             quantize_biased(v[j][6], scale), quantize_biased(v[j][7], scale));
            *reinterpret_cast<uint2 *>(qrow + 8 * vi) = make_uint2(lo, hi);
        }
    }
}

// Rows of up to 2048 elements: CTAs that walk rows blockIdx.x, blockIdx.x + gridDim.x, ... and
// request row i+1 before they work on row i; the two reduction buffers alternate from row to row,
// so each block reduction costs one barrier instead of two.  Thread t owns vector t of a row and
// the reductions run in the order of the one-row kernel: bit-identical results.  Measured on B200:
// with one row per CTA it is the fastest fused-RMSNorm quantizer below 1024 rows (the barrier it
// saves); walking many rows per CTA does not pay at 16384 rows (48 vs 40 us), so there the
// row-group kernel above is used.
template <typename T>
struct Raw8 {
    uint4 w[sizeof(T) == 4 ? 2 : 1];
    __device__ __forceinline__ void load(const T *p) {
        const uint4 *s = reinterpret_cast<const uint4 *>(p);
        w[0] = s[0];
        if (sizeof(T) == 4) w[sizeof(T) == 4 ? 1 : 0] = s[1];
    }
    __device__ __forceinline__ void zero() {
        w[0] = make_uint4(0, 0, 0, 0);
        if (sizeof(T) == 4) w[sizeof(T) == 4 ? 1 : 0] = make_uint4(0, 0, 0, 0);
    }
    __device__ __forceinline__ void unpack(float (&v)[8]) const { Load8<T>::run(w, v); }
};

template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads) quant_rows_stream_kernel(QuantArgs a) {
    __shared__ float red_f[2][kThreads / 32];
    __shared__ double red_d[2][kThreads / 32];
    pdl_trigger();
    pdl_wait();
    const int t = threadIdx.x, lane = t & 31, w = t >> 5;
    const int nvec = a.cols >> 3;
    const bool has = t < nvec;
    const T *x = reinterpret_cast<const T *>(a.x);

    Raw8<T> next;
    int row = blockIdx.x;
    if (has && row < a.rows) next.load(x + (long long)row * a.ldx + 8 * t);
    else next.zero();
    for (int it = 0; row < a.rows; row += gridDim.x, ++it) {
        const int buf = it & 1;  // the two reduction buffers alternate: one barrier per reduction
        float v[8];
        next.unpack(v);
        const int nrow = row + gridDim.x;
        if (has && nrow < a.rows) next.load(x + (long long)nrow * a.ldx + 8 * t);

        float row_factor = 1.0f;
        if (MODE == MODE_RMS) {
            double ss = 0.0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const double d = (double)v[i];
                ss = fma(d, d, ss);
            }
            ss = warp_sum(ss);
            if (lane == 0) red_d[buf][w] = ss;
            __syncthreads();
            double tot = red_d[buf][0];
#pragma unroll
            for (int i = 1; i < kThreads / 32; ++i) tot += red_d[buf][i];
            float f = 0.0f;
            if (lane == 0) f = inv_rms_of(tot, a);
            row_factor = __shfl_sync(0xffffffffu, f, 0);
        }
        float amax = 0.0f;
        if (has) {
            transform8<MODE>(v, 8 * t, a, row_factor);
#pragma unroll
            for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(v[i]));
        }
        amax = warp_max(amax);
        if (lane == 0) red_f[buf][w] = amax;
        __syncthreads();
        float m = red_f[buf][0];
#pragma unroll
        for (int i = 1; i < kThreads / 32; ++i) m = fmaxf(m, red_f[buf][i]);
        const RowScale scale = make_row_scale(m);
        if (t == 0) a.scales[row] = scale.scale;
        if (has) {
            const uint32_t lo = pack_biased4(quantize_biased(v[0], scale), quantize_biased(v[1], scale),
                                             quantize_biased(v[2], scale), quantize_biased(v[3], scale));
            const uint32_t hi = pack_biased4(quantize_biased(v[4], scale), quantize_biased(v[5], scale),
                                             quantize_biased(v[6], scale), quantize_biased(v[7], scale));
            *reinterpret_cast<uint2 *>(a.q + (long long)row * a.ldq + 8 * t) = make_uint2(lo, hi);
        }
    }
}

// General path for any width / alignment: one CTA per row, the row is re-read for each
// pass.  Only odd shapes land here.
template <typename T, int MODE>
__global__ void __launch_bounds__(kThreads) quant_rows_any_kernel(QuantArgs a) {
    __shared__ float red_f[kThreads / 32];
    __shared__ double red_d[kThreads / 32];
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.x;
    const T *xrow = reinterpret_cast<const T *>(a.x) + (long long)row * a.ldx;

    float row_factor = 1.0f;
    if (MODE == MODE_RMS) {
        double ss = 0.0;
        for (int c = threadIdx.x; c < a.cols; c += kThreads) {
            double d = (double)Load8<T>::one(xrow, c);
            ss = fma(d, d, ss);
        }
        ss = group_sum<kThreads>(ss, red_d);
        row_factor = inv_rms_of(ss, a);
    } else if (MODE == MODE_DEQ_ACT) {
        row_factor = a.in_row_scales[row];
    }
    auto value = [&](int c) -> float {
        float t = Load8<T>::one(xrow, c);
        if (MODE == MODE_RMS) {
            t = __fmul_rn(t, row_factor);
            if (a.vec_scale) t = __fmul_rn(t, a.scale_is_mod ? __fadd_rn(1.0f, a.vec_scale[c]) : a.vec_scale[c]);
            if (a.vec_bias) t = __fadd_rn(t, a.vec_bias[c]);
        } else if (MODE == MODE_DEQ_ACT) {
            t = __fmul_rn(__fmul_rn(t, row_factor), a.col_scales[c]);
            if (a.vec_bias) t = __fadd_rn(t, a.vec_bias[c]);
            t = apply_act_rt(t, a.act);
        }
        return t;
    };
    float amax = 0.0f;
    for (int c = threadIdx.x; c < a.cols; c += kThreads) amax = fmaxf(amax, fabsf(value(c)));
    amax = group_max<kThreads>(amax, red_f);
    const RowScale scale = make_row_scale(amax);
    __syncthreads();  // every thread has read in_row_scales[row] before it may be overwritten
    if (threadIdx.x == 0) a.scales[row] = scale.scale;
    int8_t *qrow = a.q + (long long)row * a.ldq;
    for (int c = threadIdx.x; c < a.cols; c += kThreads) qrow[c] = (int8_t)quantize_code(value(c), scale);
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T, int MODE>
int launch_quant(const QuantArgs &a, cudaStream_t stream) {
    if (a.rows == 0 || a.cols == 0) return 0;
    const size_t esz = sizeof(T);
    bool vec_ok = (a.cols % 8 == 0) && aligned16(a.x) && ((a.ldx * esz) % 16 == 0) &&
                  ((reinterpret_cast<uintptr_t>(a.q) & 7u) == 0) && (a.ldq % 8 == 0) &&
                  a.cols <= kThreads * 8 * kMaxVec;
    if (MODE == MODE_RMS) vec_ok = vec_ok && (!a.vec_scale || aligned16(a.vec_scale)) && (!a.vec_bias || aligned16(a.vec_bias));
    if (MODE == MODE_DEQ_ACT) vec_ok = vec_ok && aligned16(a.col_scales) && (!a.vec_bias || aligned16(a.vec_bias));
    if (!vec_ok) {
        launch_kernel(quant_rows_any_kernel<T, MODE>, dim3(a.rows), dim3(kThreads), 0, stream, a);
        return check_launch("quant_rows_any");
    }
    // Narrow rows: a warp per row (no block barriers at all).  Rows of 1024 elements or more: a
    // whole CTA per row; that keeps more bytes in flight per SM and measured faster at every
    // row count from 512 to 16384.
    const int nvec = a.cols / 8;
    const bool warp_rows = nvec <= 64 || (nvec < 128 && a.rows >= 2048);
    if (warp_rows) {
        constexpr int kRows = kThreads / 32;
        const unsigned grid = (unsigned)((a.rows + kRows - 1) / kRows);
        if (nvec <= 32) launch_kernel(quant_rows_vec_kernel<T, MODE, 32, 1>, dim3(grid), dim3(kThreads), 0, stream, a);
        else if (nvec <= 64) launch_kernel(quant_rows_vec_kernel<T, MODE, 32, 2>, dim3(grid), dim3(kThreads), 0, stream, a);
        else if (nvec <= 128) launch_kernel(quant_rows_vec_kernel<T, MODE, 32, 4>, dim3(grid), dim3(kThreads), 0, stream, a);
        else launch_kernel(quant_rows_vec_kernel<T, MODE, 32, 8>, dim3(grid), dim3(kThreads), 0, stream, a);
    } else if (nvec <= 256 && MODE == MODE_RMS && a.rows < 1024) {
        // few rows: the walking kernel with one row per CTA -- its alternating reduction buffers need
        // one block barrier per reduction instead of two (2.75 vs 3.6 us at 512 rows)
        launch_kernel(quant_rows_stream_kernel<T, MODE>, dim3((unsigned)a.rows), dim3(kThreads), 0, stream, a);
    } else if (nvec <= 256 && MODE == MODE_RMS && a.rows >= 2048) {
        // four rows per CTA, 64 threads each with four vectors: the per-thread costs (reductions, the
        // scale's division and reciprocal) are shared by 32 elements instead of 8; measured 35.5 us
        // at 16384 rows against 37.3 us for two rows per CTA and 46.5 us for a warp per row with 64
        // elements per thread
        launch_kernel(quant_rows_vec_kernel<T, MODE, 64, 4>, dim3((unsigned)((a.rows + 3) / 4)), dim3(kThreads), 0,
                      stream, a);
    } else if (nvec <= 256 && MODE == MODE_RMS && a.rows >= 1024) {
        // two rows per CTA, 128 threads each (faster than four rows per CTA at 1024 rows: 4.6 vs 5.9 us)
        launch_kernel(quant_rows_vec_kernel<T, MODE, 128, 2>, dim3((unsigned)((a.rows + 1) / 2)), dim3(kThreads), 0,
                      stream, a);
    } else {
        const unsigned grid = (unsigned)a.rows;
        if (nvec <= 256) launch_kernel(quant_rows_vec_kernel<T, MODE, kThreads, 1>, dim3(grid), dim3(kThreads), 0, stream, a);
        else if (nvec <= 512) launch_kernel(quant_rows_vec_kernel<T, MODE, kThreads, 2>, dim3(grid), dim3(kThreads), 0, stream, a);
        else if (nvec <= 1024) launch_kernel(quant_rows_vec_kernel<T, MODE, kThreads, 4>, dim3(grid), dim3(kThreads), 0, stream, a);
        else launch_kernel(quant_rows_vec_kernel<T, MODE, kThreads, 8>, dim3(grid), dim3(kThreads), 0, stream, a);
    }
    return check_launch("quant_rows_vec");
}

template <int MODE>
int dispatch_in_dtype(int in_dtype, const QuantArgs &a, cudaStream_t stream) {
    switch (in_dtype) {
        case B200_DT_F32: return launch_quant<float, MODE>(a, stream);
        case B200_DT_F16: return launch_quant<__half, MODE>(a, stream);
        case B200_DT_BF16: return launch_quant<__nv_bfloat16, MODE>(a, stream);
        default: return fail("unsupported activation dtype %d", in_dtype);
    }
}

}  // namespace

int quantize_rows(const void *x, int in_dtype, long long ldx, int8_t *q, long long ldq, float *scales, int rows,
                  int cols, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return 0;
    if (!x || !q || !scales || rows < 0 || cols < 0 || ldx < cols || ldq < cols)
        return fail("invalid quantize_rows arguments rows=%d cols=%d", rows, cols);
    QuantArgs a{};
    a.x = x; a.ldx = ldx; a.q = q; a.ldq = ldq; a.scales = scales; a.rows = rows; a.cols = cols;
    return dispatch_in_dtype<MODE_PLAIN>(in_dtype, a, stream);
}

int rms_norm_quantize_rows(const void *x, int in_dtype, long long ldx, const float *vec_scale, int scale_is_mod,
                           const float *vec_bias, int8_t *q, long long ldq, float *scales, int rows, int cols,
                           float eps, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return 0;
    if (!x || !q || !scales || rows < 0 || cols < 0 || ldx < cols || ldq < cols)
        return fail("invalid rms_norm_quantize_rows arguments rows=%d cols=%d", rows, cols);
    QuantArgs a{};
    a.x = x; a.ldx = ldx; a.q = q; a.ldq = ldq; a.scales = scales; a.rows = rows; a.cols = cols;
    a.vec_scale = vec_scale; a.vec_bias = vec_bias; a.scale_is_mod = scale_is_mod; a.eps = eps;
    a.inv_cols = (cols & (cols - 1)) == 0 ? 1.0 / (double)cols : 0.0;
    return dispatch_in_dtype<MODE_RMS>(in_dtype, a, stream);
}

int dequant_act_quantize_rows(const int32_t *acc, long long ldacc, const float *in_row_scales,
                              const float *col_scales, const float *bias, int act, int8_t *q, long long ldq,
                              float *out_row_scales, int rows, int cols, cudaStream_t stream) {
    if (rows == 0 || cols == 0) return 0;
    if (!acc || !in_row_scales || !col_scales || !q || !out_row_scales || rows < 0 || cols < 0 || ldacc < cols ||
        ldq < cols || act < 0 || act > 2)
        return fail("invalid dequant_act_quantize_rows arguments rows=%d cols=%d act=%d", rows, cols, act);
    QuantArgs a{};
    a.x = acc; a.ldx = ldacc; a.q = q; a.ldq = ldq; a.scales = out_row_scales; a.rows = rows; a.cols = cols;
    a.in_row_scales = in_row_scales; a.col_scales = col_scales; a.vec_bias = bias; a.act = act;
    return launch_quant<int32_t, MODE_DEQ_ACT>(a, stream);
}

}  // namespace b200
