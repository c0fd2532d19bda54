// Stand-alone consumers of an int32 accumulator: dequant (+gate) + residual, and the QKV
// dequant + per-head RMSNorm + RoPE.  They exist so that a caller which keeps the
// reference's three-call sequence (quantize -> int32 GEMM -> dequant) keeps working; the
// fused linear makes the first of them unnecessary.  Both are pure HBM-bandwidth kernels:
// 4 B/element of accumulator in, residual in, result out.
#include <math.h>

#include "common.cuh"
#include "w8a8_internal.h"

namespace b200 {

namespace {

template <typename T>
struct Elem;
template <>
struct Elem<float> {
    static __device__ __forceinline__ void load4(const void *p, float (&v)[4]) {
        float4 a = *reinterpret_cast<const float4 *>(p);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    }
    static __device__ __forceinline__ void store4(void *p, const float (&v)[4]) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
    static __device__ __forceinline__ float load1(const void *p, long long i) {
        return reinterpret_cast<const float *>(p)[i];
    }
    static __device__ __forceinline__ void store1(void *p, long long i, float v) {
        reinterpret_cast<float *>(p)[i] = v;
    }
};
template <>
struct Elem<__half> {
    static __device__ __forceinline__ void load4(const void *p, float (&v)[4]) {
        uint2 raw = *reinterpret_cast<const uint2 *>(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&raw);
        float2 a = __half22float2(h[0]), b = __half22float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store4(void *p, const float (&v)[4]) {
        __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t *>(&a);
        raw.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(p) = raw;
    }
    static __device__ __forceinline__ float load1(const void *p, long long i) {
        return __half2float(reinterpret_cast<const __half *>(p)[i]);
    }
    static __device__ __forceinline__ void store1(void *p, long long i, float v) {
        reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    }
};
template <>
struct Elem<__nv_bfloat16> {
    static __device__ __forceinline__ void load4(const void *p, float (&v)[4]) {
        uint2 raw = *reinterpret_cast<const uint2 *>(p);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&raw);
        float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store4(void *p, const float (&v)[4]) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t *>(&a);
        raw.y = *reinterpret_cast<uint32_t *>(&b);
        *reinterpret_cast<uint2 *>(p) = raw;
    }
    static __device__ __forceinline__ float load1(const void *p, long long i) {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    }
    static __device__ __forceinline__ void store1(void *p, long long i, float v) {
        reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    }
};

// One thread per 4 consecutive columns; the 2-D grid removes the per-element integer divide.
template <typename TR, typename TO, bool VEC>
__global__ void __launch_bounds__(256) dequant_residual_kernel(
    const int32_t *__restrict__ acc, const float *__restrict__ row_scales, const float *__restrict__ col_scales,
    const void *__restrict__ residual, const float *__restrict__ gate, void *__restrict__ out, int rows, int cols) {
    pdl_trigger();
    pdl_wait();
    const int row = blockIdx.y;
    const float rs = row_scales[row];
    const long long base = (long long)row * cols;
    if (VEC) {
        const int c = (blockIdx.x * 256 + threadIdx.x) * 4;
        if (c >= cols) return;
        int4 a = *reinterpret_cast<const int4 *>(acc + base + c);
        float4 cs = *reinterpret_cast<const float4 *>(col_scales + c);
        float v[4] = {dequant_acc(a.x, rs, cs.x), dequant_acc(a.y, rs, cs.y), dequant_acc(a.z, rs, cs.z),
                      dequant_acc(a.w, rs, cs.w)};
        if (gate) {
            float4 g = *reinterpret_cast<const float4 *>(gate + c);
            v[0] = __fmul_rn(v[0], g.x); v[1] = __fmul_rn(v[1], g.y);
            v[2] = __fmul_rn(v[2], g.z); v[3] = __fmul_rn(v[3], g.w);
        }
        if (residual) {
            float r[4];
            Elem<TR>::load4(reinterpret_cast<const TR *>(residual) + base + c, r);
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = __fadd_rn(r[i], v[i]);
        }
        Elem<TO>::store4(reinterpret_cast<TO *>(out) + base + c, v);
    } else {
        const int c = blockIdx.x * 256 + threadIdx.x;
        if (c >= cols) return;
        float v = dequant_acc(acc[base + c], rs, col_scales[c]);
        if (gate) v = __fmul_rn(v, gate[c]);
        if (residual) v = __fadd_rn(Elem<TR>::load1(residual, base + c), v);
        Elem<TO>::store1(out, base + c, v);
    }
}

bool aligned16(const void *p) { return !p || (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename TR, typename TO>
int launch_dequant_residual(const int32_t *acc, const float *rs, const float *cs, const void *res,
                            const float *gate, void *out, int rows, int cols, cudaStream_t stream) {
    const bool vec = (cols % 4 == 0) && aligned16(acc) && aligned16(cs) && aligned16(res) && aligned16(gate) &&
                     aligned16(out);
    if (vec) {
        dim3 grid((cols / 4 + 255) / 256, rows);
        launch_kernel(dequant_residual_kernel<TR, TO, true>, grid, dim3(256), 0, stream, acc, rs, cs, res, gate, out, rows, cols);
    } else {
        dim3 grid((cols + 255) / 256, rows);
        launch_kernel(dequant_residual_kernel<TR, TO, false>, grid, dim3(256), 0, stream, acc, rs, cs, res, gate, out, rows, cols);
    }
    return check_launch("dequant_residual");
}

// Phase of rotary pair `pair_id`: x and y positions are mapped to pixel centres in [-1,1]
// and use the shared xy frequency table; the rest of the pairs rotate with time.
__device__ __forceinline__ float rope_phase(int pair_id, long long x_pos, long long y_pos, long long t_pos,
                                            const float *xy, const float *inv_t, int width, int height, int d_xy) {
    if (pair_id < d_xy) {
        float x = __fsub_rn(__fdiv_rn(__fadd_rn(__fmul_rn(2.0f, (float)x_pos), 1.0f), (float)width), 1.0f);
        return __fmul_rn(x, xy[pair_id]);
    }
    if (pair_id < 2 * d_xy) {
        float y = __fsub_rn(__fdiv_rn(__fadd_rn(__fmul_rn(2.0f, (float)y_pos), 1.0f), (float)height), 1.0f);
        return __fmul_rn(y, xy[pair_id - d_xy]);
    }
    return __fmul_rn((float)t_pos, inv_t[pair_id - 2 * d_xy]);
}

// One warp per (token, head role).  The head's d_head values are dequantized once into
// registers (lane owns pairs lane, lane+32, ...), reduced with shuffles, rotated and
// written head-major.  The reference spends a 256-thread CTA and 2 barriers per head.
constexpr int kMaxPairsPerLane = 4;  // d_head <= 256

__global__ void __launch_bounds__(256) qkv_rms_rope_dequant_kernel(
    const int32_t *__restrict__ qkv_acc, const float *__restrict__ row_scales,
    const float *__restrict__ weight_scales, float *__restrict__ q, float *__restrict__ k, float *__restrict__ v,
    const int64_t *__restrict__ x_pos, const int64_t *__restrict__ y_pos, const int64_t *__restrict__ t_pos,
    const float *__restrict__ xy, const float *__restrict__ inv_t, int T, int n_heads, int n_kv_heads, int d_head,
    int width, int height, float eps) {
    pdl_trigger();
    pdl_wait();
    const int roles = n_heads + 2 * n_kv_heads;
    const long long unit = (long long)blockIdx.x * 8 + (threadIdx.x >> 5);
    if (unit >= (long long)T * roles) return;
    const int t = (int)(unit / roles);
    const int role = (int)(unit - (long long)t * roles);
    const int lane = threadIdx.x & 31;
    const int q_dim = n_heads * d_head, kv_dim = n_kv_heads * d_head;
    const int half = d_head / 2, d_xy = d_head / 8;
    const int32_t *row = qkv_acc + (long long)t * (q_dim + 2 * kv_dim);
    const float rs = row_scales[t];

    if (role < n_heads + n_kv_heads) {
        const bool is_k = role >= n_heads;
        const int h = is_k ? role - n_heads : role;
        const int base = is_k ? q_dim + h * d_head : h * d_head;
        float a[kMaxPairsPerLane], b[kMaxPairsPerLane];
        double ss = 0.0;
#pragma unroll
        for (int j = 0; j < kMaxPairsPerLane; ++j) {
            int p = lane + 32 * j;
            a[j] = b[j] = 0.0f;
            if (p < half) {
                int2 raw = *reinterpret_cast<const int2 *>(row + base + 2 * p);
                float2 ws = *reinterpret_cast<const float2 *>(weight_scales + base + 2 * p);
                a[j] = dequant_acc(raw.x, rs, ws.x);
                b[j] = dequant_acc(raw.y, rs, ws.y);
                ss = fma((double)a[j], (double)a[j], ss);
                ss = fma((double)b[j], (double)b[j], ss);
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = (float)(1.0 / sqrt(ss / (double)d_head + (double)eps));
        float *dst = (is_k ? k : q) + ((long long)h * T + t) * d_head;
        const long long xp = x_pos[t], yp = y_pos[t], tp = t_pos[t];
#pragma unroll
        for (int j = 0; j < kMaxPairsPerLane; ++j) {
            int p = lane + 32 * j;
            if (p < half) {
                float phase = rope_phase(p, xp, yp, tp, xy, inv_t, width, height, d_xy);
                float c = cosf(phase), s = sinf(phase);
                float an = __fmul_rn(a[j], inv), bn = __fmul_rn(b[j], inv);
                dst[p] = __fsub_rn(__fmul_rn(an, c), __fmul_rn(bn, s));
                dst[half + p] = __fadd_rn(__fmul_rn(bn, c), __fmul_rn(an, s));
            }
        }
    } else {
        const int h = role - n_heads - n_kv_heads;
        const int base = q_dim + kv_dim + h * d_head;
        float *dst = v + ((long long)h * T + t) * d_head;
        for (int d = lane; d < d_head; d += 32) dst[d] = dequant_acc(row[base + d], rs, weight_scales[base + d]);
    }
}

// cos / sin of every (token, rotary pair): the values the QKV consumer would compute per head,
// computed once per frame (positions do not change from layer to layer).
__global__ void __launch_bounds__(256) rope_tables_kernel(const int64_t *__restrict__ x_pos,
                                                          const int64_t *__restrict__ y_pos,
                                                          const int64_t *__restrict__ t_pos,
                                                          const float *__restrict__ xy, const float *__restrict__ inv_t,
                                                          int T, int half, int d_xy, int width, int height,
                                                          float *__restrict__ cos_out, float *__restrict__ sin_out) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)T * half) return;
    const int t = (int)(i / half), pair = (int)(i - (long long)t * half);
    const float phase = rope_phase(pair, x_pos[t], y_pos[t], t_pos[t], xy, inv_t, width, height, d_xy);
    cos_out[i] = cosf(phase);
    sin_out[i] = sinf(phase);
}

}  // namespace

int rope_tables(const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos, const float *xy, const float *inv_t,
                int tokens, int d_head, int width, int height, float *cos_out, float *sin_out, cudaStream_t stream) {
    if (!x_pos || !y_pos || !t_pos || !xy || !inv_t || !cos_out || !sin_out || tokens < 0 || d_head <= 0 ||
        width <= 0 || height <= 0 || d_head % 8 != 0)
        return fail("invalid rope_tables arguments tokens=%d d_head=%d", tokens, d_head);
    if (tokens == 0) return 0;
    const long long n = (long long)tokens * (d_head / 2);
    launch_kernel(rope_tables_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, x_pos, y_pos, t_pos, xy,
                  inv_t, tokens, d_head / 2, d_head / 8, width, height, cos_out, sin_out);
    return check_launch("rope_tables");
}

int dequant_residual(const int32_t *acc, const float *row_scales, const float *col_scales, const void *residual,
                     int res_dtype, const float *gate, void *out, int out_dtype, int rows, int cols,
                     cudaStream_t stream) {
    if (rows == 0 || cols == 0) return 0;
    if (!acc || !row_scales || !col_scales || !out || rows < 0 || cols < 0)
        return fail("invalid dequant_residual arguments rows=%d cols=%d", rows, cols);
    if (rows > 65535 * 1) {
        // grid.y limit: split into slabs of rows
        const int step = 65535;
        for (int r0 = 0; r0 < rows; r0 += step) {
            int nr = rows - r0 < step ? rows - r0 : step;
            size_t esz_r = res_dtype == B200_DT_F32 ? 4 : 2, esz_o = out_dtype == B200_DT_F32 ? 4 : 2;
            const void *res = residual ? (const char *)residual + (size_t)r0 * cols * esz_r : nullptr;
            if (dequant_residual(acc + (size_t)r0 * cols, row_scales + r0, col_scales, res, res_dtype, gate,
                                 (char *)out + (size_t)r0 * cols * esz_o, out_dtype, nr, cols, stream))
                return 1;
        }
        return 0;
    }
    if (!residual) res_dtype = out_dtype;
#define B200_DR(TR, TO) \
    return launch_dequant_residual<TR, TO>(acc, row_scales, col_scales, residual, gate, out, rows, cols, stream)
    if (res_dtype == B200_DT_F32 && out_dtype == B200_DT_F32) B200_DR(float, float);
    if (res_dtype == B200_DT_F16 && out_dtype == B200_DT_F16) B200_DR(__half, __half);
    if (res_dtype == B200_DT_BF16 && out_dtype == B200_DT_BF16) B200_DR(__nv_bfloat16, __nv_bfloat16);
    if (res_dtype == B200_DT_F32 && out_dtype == B200_DT_F16) B200_DR(float, __half);
    if (res_dtype == B200_DT_F32 && out_dtype == B200_DT_BF16) B200_DR(float, __nv_bfloat16);
#undef B200_DR
    return fail("unsupported dequant_residual dtypes residual=%d out=%d", res_dtype, out_dtype);
}

int qkv_rms_rope_dequant(const int32_t *qkv_acc, const float *row_scales, const float *weight_scales, float *q,
                         float *k, float *v, const int64_t *x_pos, const int64_t *y_pos, const int64_t *t_pos,
                         const float *xy, const float *inv_t, int tokens, int n_heads, int n_kv_heads, int d_head,
                         int width, int height, float eps, cudaStream_t stream) {
    if (!qkv_acc || !row_scales || !weight_scales || !q || !k || !v || !x_pos || !y_pos || !t_pos || !xy ||
        !inv_t || tokens < 0 || n_heads <= 0 || n_kv_heads <= 0 || d_head <= 0 || width <= 0 || height <= 0)
        return fail("invalid qkv_rms_rope_dequant arguments");
    if (d_head % 8 != 0 || d_head > 64 * kMaxPairsPerLane)
        return fail("qkv_rms_rope_dequant needs d_head %% 8 == 0 and d_head <= %d, got %d", 64 * kMaxPairsPerLane,
                    d_head);
    if (tokens == 0) return 0;
    // the kernel reads accumulators and weight scales two at a time
    if (((reinterpret_cast<uintptr_t>(qkv_acc) | reinterpret_cast<uintptr_t>(weight_scales)) & 7u) != 0)
        return fail("qkv_rms_rope_dequant needs 8-byte aligned qkv_acc and weight_scales");
    const long long units = (long long)tokens * (n_heads + 2 * n_kv_heads);
    launch_kernel(qkv_rms_rope_dequant_kernel, dim3((unsigned)((units + 7) / 8)), dim3(256), 0, stream, qkv_acc,
                  row_scales, weight_scales, q, k, v, x_pos, y_pos, t_pos, xy, inv_t, tokens, n_heads, n_kv_heads,
                  d_head, width, height, eps);
    return check_launch("qkv_rms_rope_dequant");
}

}  // namespace b200
