// s8 x s8 -> s32 GEMM for sm_100a with the epilogue of a W8A8 linear fused in.
//
//   acc[m,n] = sum_k x[m,k] * w[n,k]          x: int8 [M,K] row-major, w: int8 [N,K]
//   y[m,n]   = residual + gate * act(acc * sx[m] * sw[n] + bias[n])      (optional parts)
//
// It replaces the reference's CUTLASS Ampere-class mma.sync instantiation and the
// separate dequant kernels that re-read its int32 scratch
// (src/world_cuda_ops.cu:529-599, 229-262).
//
// Structure: a persistent kernel, one CTA per SM, 192 threads in three roles.
//   warp 0    : TMA producer.  Streams 128-row x 128-byte operand slabs of A and W into a
//               ring of shared-memory stages (128-byte swizzle), signalling `full` mbarriers.
//   warp 1    : MMA issuer.  One thread issues tcgen05.mma (kind i8, 128 x BN x 32 per
//               instruction, four per stage) into one of two TMEM accumulators and commits
//               completion to the stage's `empty` barrier / the accumulator's `full` barrier.
//   warps 2-5 : epilogue.  Each owns one 32-lane TMEM sub-partition (= 32 rows of the tile),
//               pulls accumulators out with tcgen05.ld, applies the fused epilogue in
//               registers and stores.  The second accumulator lets tile i+1's main loop
//               run under tile i's epilogue.
// Both operands are K-major in memory already, so nothing is transposed; the operand
// descriptors only differ in height.  Every wait is bounded (see mbar_wait_bounded): on
// expiry the CTA drains and the kernel leaves a status word instead of hanging.
//
// Roofline: tensor-bound for M >= ~1024 (2*M*N*K ops), HBM-bound on the N*K weight bytes
// for M <= 128.
#include <cuda.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "w8a8_internal.h"

namespace b200 {

__device__ int g_gemm_status = 0;

namespace {

constexpr int BM = 128;       // rows per tile = TMEM lanes
constexpr int BK = 128;       // bytes of K per pipeline stage = one swizzle atom
constexpr int kThreads = 192;
constexpr int kSmemBudget = 200 * 1024;

template <int BN>
struct Cfg {
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kStages = kSmemBudget / kStageBytes > 10 ? 10 : kSmemBudget / kStageBytes;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;  // + alignment slack
};

struct GemmParams {
    int M, N, K;
    int num_m_blocks, num_n_blocks, num_tiles, num_k_blocks;
    int group_m;     // m-blocks per raster group (keeps a band of A resident in L2)
    int b_kx, b_kz;  // W coordinate multipliers: row-major (128,0), slab layout (0,1)
    const float *row_scales;
    const float *col_scales;
    const float *bias;
    const float *gate;
    const void *residual;
    long long ldr;
    void *out;
    long long ldo;
    int out_dtype;
    int act;
    int vec_ok;  // 16-byte vector stores/loads are legal for out / residual
};

__device__ __forceinline__ void decode_tile(const GemmParams &p, int tile, int &m_blk, int &n_blk) {
    const int per_group = p.group_m * p.num_n_blocks;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int gm0 = g * p.group_m;
    const int gsize = min(p.group_m, p.num_m_blocks - gm0);
    n_blk = r / gsize;
    m_blk = gm0 + (r - n_blk * gsize);
}

// Stores 32 consecutive columns of one row.  v holds raw accumulators (as bit patterns).
template <int BN>
__device__ __forceinline__ void epilogue_chunk(const GemmParams &p, const uint32_t (&r)[32], int row, int col0,
                                               float row_scale) {
    const bool full = (col0 + 32 <= p.N) && p.vec_ok;
    if (p.out_dtype == B200_DT_S32) {
        int32_t *dst = reinterpret_cast<int32_t *>(p.out) + (long long)row * p.ldo + col0;
        if (full) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
                reinterpret_cast<int4 *>(dst)[g] = make_int4((int)r[4 * g], (int)r[4 * g + 1], (int)r[4 * g + 2],
                                                             (int)r[4 * g + 3]);
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j)
                if (col0 + j < p.N) dst[j] = (int)r[j];
        }
        return;
    }

    float v[32];
    if (full) {
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            float4 cs = __ldg(reinterpret_cast<const float4 *>(p.col_scales + col0) + g);
            v[4 * g + 0] = dequant_acc((int)r[4 * g + 0], row_scale, cs.x);
            v[4 * g + 1] = dequant_acc((int)r[4 * g + 1], row_scale, cs.y);
            v[4 * g + 2] = dequant_acc((int)r[4 * g + 2], row_scale, cs.z);
            v[4 * g + 3] = dequant_acc((int)r[4 * g + 3], row_scale, cs.w);
        }
        if (p.bias) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                float4 b = __ldg(reinterpret_cast<const float4 *>(p.bias + col0) + g);
                v[4 * g + 0] = __fadd_rn(v[4 * g + 0], b.x);
                v[4 * g + 1] = __fadd_rn(v[4 * g + 1], b.y);
                v[4 * g + 2] = __fadd_rn(v[4 * g + 2], b.z);
                v[4 * g + 3] = __fadd_rn(v[4 * g + 3], b.w);
            }
        }
        if (p.act != B200_ACT_NONE) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = apply_act_rt(v[j], p.act);
        }
        if (p.gate) {
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                float4 b = __ldg(reinterpret_cast<const float4 *>(p.gate + col0) + g);
                v[4 * g + 0] = __fmul_rn(v[4 * g + 0], b.x);
                v[4 * g + 1] = __fmul_rn(v[4 * g + 1], b.y);
                v[4 * g + 2] = __fmul_rn(v[4 * g + 2], b.z);
                v[4 * g + 3] = __fmul_rn(v[4 * g + 3], b.w);
            }
        }
        if (p.out_dtype == B200_DT_F32) {
            float *dst = reinterpret_cast<float *>(p.out) + (long long)row * p.ldo + col0;
            if (p.residual) {
                const float4 *res =
                    reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.residual) +
                                                     (long long)row * p.ldr + col0);
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    float4 a = res[g];
                    v[4 * g + 0] = __fadd_rn(a.x, v[4 * g + 0]);
                    v[4 * g + 1] = __fadd_rn(a.y, v[4 * g + 1]);
                    v[4 * g + 2] = __fadd_rn(a.z, v[4 * g + 2]);
                    v[4 * g + 3] = __fadd_rn(a.w, v[4 * g + 3]);
                }
            }
#pragma unroll
            for (int g = 0; g < 8; ++g)
                reinterpret_cast<float4 *>(dst)[g] = make_float4(v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
        } else {
            // 16-bit outputs: 32 columns = 64 bytes = four 16-byte vectors
            uint16_t *dst = reinterpret_cast<uint16_t *>(p.out) + (long long)row * p.ldo + col0;
            const bool is_half = p.out_dtype == B200_DT_F16;
            if (p.residual) {
                const uint4 *res = reinterpret_cast<const uint4 *>(
                    reinterpret_cast<const uint16_t *>(p.residual) + (long long)row * p.ldr + col0);
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 raw = res[g];
                    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float2 f = is_half ? __half22float2(*reinterpret_cast<const __half2 *>(&w[i]))
                                           : __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w[i]));
                        v[8 * g + 2 * i] = __fadd_rn(f.x, v[8 * g + 2 * i]);
                        v[8 * g + 2 * i + 1] = __fadd_rn(f.y, v[8 * g + 2 * i + 1]);
                    }
                }
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                uint32_t w[4];
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (is_half) {
                        __half2 h = __floats2half2_rn(v[8 * g + 2 * i], v[8 * g + 2 * i + 1]);
                        w[i] = *reinterpret_cast<uint32_t *>(&h);
                    } else {
                        __nv_bfloat162 h = __floats2bfloat162_rn(v[8 * g + 2 * i], v[8 * g + 2 * i + 1]);
                        w[i] = *reinterpret_cast<uint32_t *>(&h);
                    }
                }
                reinterpret_cast<uint4 *>(dst)[g] = make_uint4(w[0], w[1], w[2], w[3]);
            }
        }
        return;
    }

    // ragged edge or unaligned buffers: one element at a time
#pragma unroll 1
    for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col >= p.N) break;
        float t = dequant_acc((int)r[j], row_scale, p.col_scales[col]);
        if (p.bias) t = __fadd_rn(t, p.bias[col]);
        t = apply_act_rt(t, p.act);
        if (p.gate) t = __fmul_rn(t, p.gate[col]);
        const long long oi = (long long)row * p.ldo + col, ri = (long long)row * p.ldr + col;
        if (p.out_dtype == B200_DT_F32) {
            if (p.residual) t = __fadd_rn(reinterpret_cast<const float *>(p.residual)[ri], t);
            reinterpret_cast<float *>(p.out)[oi] = t;
        } else if (p.out_dtype == B200_DT_F16) {
            if (p.residual) t = __fadd_rn(__half2float(reinterpret_cast<const __half *>(p.residual)[ri]), t);
            reinterpret_cast<__half *>(p.out)[oi] = __float2half_rn(t);
        } else {
            if (p.residual)
                t = __fadd_rn(__bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p.residual)[ri]), t);
            reinterpret_cast<__nv_bfloat16 *>(p.out)[oi] = __float2bfloat16_rn(t);
        }
    }
}

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_i8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const GemmParams p) {
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(smem + C::kStages * C::kStageBytes);
    uint64_t *bar_empty = bar_full + C::kStages;
    uint64_t *bar_tfull = bar_empty + C::kStages;
    uint64_t *bar_tempty = bar_tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_tempty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_tfull[b], 1);
            mbar_init(&bar_tempty[b], 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                int m_blk, n_blk;
                decode_tile(p, tile, m_blk, n_blk);
                const int m0 = m_blk * BM, n0 = n_blk * BN;
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    ok = mbar_wait_bounded(&bar_empty[s], ph ^ 1u, abort_flag, &g_gemm_status, KS_TIMEOUT_SMEM_EMPTY);
                    if (!ok) break;
                    uint8_t *sa = smem + s * C::kStageBytes;
                    mbar_arrive_expect_tx(&bar_full[s], C::kStageBytes);
                    tma_load_3d(sa, &tm_a, &bar_full[s], kb * BK, m0, 0);
                    tma_load_3d(sa + C::kABytes, &tm_b, &bar_full[s], kb * p.b_kx, n0, kb * p.b_kz);
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(BM, BN);
            int s = 0;
            uint32_t ph = 0;
            int t = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++t) {
                const int b = t & 1;
                const uint32_t tph = (uint32_t)(t >> 1) & 1u;
                ok = mbar_wait_bounded(&bar_tempty[b], tph ^ 1u, abort_flag, &g_gemm_status, KS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    ok = mbar_wait_bounded(&bar_full[s], ph, abort_flag, &g_gemm_status, KS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * C::kStageBytes);
                    const uint64_t da = umma_smem_desc_k128(sa);
                    const uint64_t db = umma_smem_desc_k128(sa + C::kABytes);
#pragma unroll
                    for (int j = 0; j < BK / 32; ++j)
                        umma_i8(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (uint32_t)((kb | j) != 0));
                    umma_commit(&bar_empty[s]);
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(&bar_tfull[b]);
            }
        }
    } else {
        const int sub = warp & 3;  // TMEM sub-partition this warp may read
        int t = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x, ++t) {
            int m_blk, n_blk;
            decode_tile(p, tile, m_blk, n_blk);
            const int b = t & 1;
            const uint32_t tph = (uint32_t)(t >> 1) & 1u;
            ok = mbar_wait_bounded(&bar_tfull[b], tph, abort_flag, &g_gemm_status, KS_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const int row = m_blk * BM + sub * 32 + lane;
            const bool row_live = row < p.M;
            const float row_scale = (row_live && p.out_dtype != B200_DT_S32) ? p.row_scales[row] : 0.0f;
            const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(b * BN);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                tmem_ld_wait();
                const int col0 = n_blk * BN + c * 32;
                if (row_live && col0 < p.N) epilogue_chunk<BN>(p, r, row, col0, row_scale);
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_tempty[b]);
        }
    }

    __syncthreads();
    if (*abort_flag) {
        // a wait ran out somewhere: give copies and MMAs already in flight time to land
        // before the shared and tensor memory they target is released
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// A byte matrix seen as (inner 128-byte run, rows, slabs) with the 128-byte swizzle.
int make_map(CUtensorMap *map, const void *base, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1,
             uint64_t stride2, uint32_t box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {BK, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void *>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
        return fail("cuTensorMapEncodeTiled failed (%d) dims=%llu,%llu,%llu strides=%llu,%llu box_rows=%u", (int)r,
                    (unsigned long long)d0, (unsigned long long)d1, (unsigned long long)d2,
                    (unsigned long long)stride1, (unsigned long long)stride2, box_rows);
    return 0;
}

struct DeviceInfo {
    int sms = 0;
    bool attr_set[3] = {false, false, false};
};
DeviceInfo &device_info(int dev) {
    static DeviceInfo info[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo &d = info[dev & 63];
    if (d.sms == 0) cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    return d;
}

template <int BN>
int launch_bn(const LinearArgs &a, GemmParams &p, int slot, cudaStream_t stream) {
    using C = Cfg<BN>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    DeviceInfo &di = device_info(dev);
    if (!di.attr_set[slot]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_i8_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             C::kSmemBytes);
        if (e != cudaSuccess) return fail("cudaFuncSetAttribute(smem=%d): %s", C::kSmemBytes, cudaGetErrorString(e));
        di.attr_set[slot] = true;
    }
    p.num_m_blocks = (a.m + BM - 1) / BM;
    p.num_n_blocks = (a.n + BN - 1) / BN;
    p.num_tiles = p.num_m_blocks * p.num_n_blocks;
    p.num_k_blocks = (a.k + BK - 1) / BK;
    p.group_m = 32;

    CUtensorMap tm_a, tm_b;
    if (make_map(&tm_a, a.x, (uint64_t)a.k, (uint64_t)a.m, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.m, BM))
        return 1;
    if (a.w_layout == B200_W_SLAB128) {
        if (make_map(&tm_b, a.w, BK, (uint64_t)a.n, (uint64_t)(a.k / BK), BK, (uint64_t)a.n * BK, BN)) return 1;
        p.b_kx = 0;
        p.b_kz = 1;
    } else {
        if (make_map(&tm_b, a.w, (uint64_t)a.k, (uint64_t)a.n, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.n, BN))
            return 1;
        p.b_kx = BK;
        p.b_kz = 0;
    }
    const int grid = p.num_tiles < di.sms ? p.num_tiles : di.sms;
    gemm_i8_kernel<BN><<<grid, kThreads, C::kSmemBytes, stream>>>(tm_a, tm_b, p);
    return check_launch("gemm_i8_tcgen05");
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace

int gemm_can_implement(const LinearArgs &a, bool verbose) {
    auto no = [&](const char *why) {
        if (verbose) return fail("INT8 GEMM M=%d K=%d N=%d cannot run: %s", a.m, a.k, a.n, why);
        return 1;
    };
    if (!a.x || !a.w || !a.out || a.m <= 0 || a.k <= 0 || a.n <= 0) return no("invalid arguments");
    if ((a.k & 31) != 0) return no("K must be divisible by 32");
    if (!aligned16(a.x) || !aligned16(a.w)) return no("x and w must be 16-byte aligned");
    if (a.w_layout == B200_W_SLAB128 && (a.k % BK) != 0) return no("the slab weight layout needs K % 128 == 0");
    if (a.w_layout != B200_W_SLAB128 && a.w_layout != B200_W_ROW_MAJOR) return no("unknown weight layout");
    if (a.out_dtype != B200_DT_S32) {
        if (!a.row_scales || !a.col_scales) return no("row and column scales are required");
        if (a.out_dtype != B200_DT_F32 && a.out_dtype != B200_DT_F16 && a.out_dtype != B200_DT_BF16)
            return no("unsupported output dtype");
        if (a.act < 0 || a.act > 2) return no("unknown activation");
    }
    if (a.ldo < a.n || (a.residual && a.ldr < a.n)) return no("row stride smaller than N");
    return 0;
}

size_t gemm_workspace_size(int, int, int) { return 0; }

int gemm_launch(const LinearArgs &a, void *, size_t, cudaStream_t stream) {
    if (gemm_can_implement(a, true)) return 1;
    GemmParams p{};
    p.M = a.m; p.N = a.n; p.K = a.k;
    p.row_scales = a.row_scales; p.col_scales = a.col_scales; p.bias = a.bias; p.gate = a.gate;
    p.residual = a.residual; p.ldr = a.ldr; p.out = a.out; p.ldo = a.ldo;
    p.out_dtype = a.out_dtype; p.act = a.out_dtype == B200_DT_S32 ? 0 : a.act;
    const size_t esz = (a.out_dtype == B200_DT_S32 || a.out_dtype == B200_DT_F32) ? 4 : 2;
    p.vec_ok = aligned16(a.out) && ((a.ldo * esz) % 16 == 0) &&
               (!a.residual || (aligned16(a.residual) && ((a.ldr * esz) % 16 == 0))) &&
               (a.out_dtype == B200_DT_S32 ||
                (aligned16(a.col_scales) && (!a.bias || aligned16(a.bias)) && (!a.gate || aligned16(a.gate))));

    // Tile width: the widest tile is the most efficient per MMA, but a grid that leaves
    // most SMs idle loses more.  Cost model: waves x width.
    int dev = 0;
    cudaGetDevice(&dev);
    const int sms = device_info(dev).sms > 0 ? device_info(dev).sms : 148;
    const int mb = (a.m + BM - 1) / BM;
    int best_bn = 256;
    long long best_cost = -1;
    const int widths[3] = {256, 128, 64};
    for (int i = 0; i < 3; ++i) {
        const int bn = widths[i];
        const long long tiles = (long long)mb * ((a.n + bn - 1) / bn);
        const long long waves = (tiles + sms - 1) / sms;
        // relative time of one K-slab: N=64 MMAs are limited by re-reading the A operand
        // from shared memory, so they cost more than a quarter of an N=256 MMA
        const long long cost = waves * ((bn == 64 ? 96 : bn) + 16);  // +16: fixed per-tile overhead
        if (best_cost < 0 || cost < best_cost) {
            best_cost = cost;
            best_bn = bn;
        }
    }
    if (best_bn == 256) return launch_bn<256>(a, p, 0, stream);
    if (best_bn == 128) return launch_bn<128>(a, p, 1, stream);
    return launch_bn<64>(a, p, 2, stream);
}

int gemm_poll_status(int *status_out) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail("cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int st = 0;
    e = cudaMemcpyFromSymbol(&st, g_gemm_status, sizeof(int));
    if (e != cudaSuccess) return fail("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (status_out) *status_out = st;
    if (st != 0) {
        int zero = 0;
        cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    }
    return 0;
}

}  // namespace b200
