// Pieces shared by the tcgen05 GEMM translation units: tile configuration, the kernel
// parameter block, the fp32 epilogue arithmetic, the staged TMA store of output blocks and the
// host-side tensor-map helpers.  Everything lives in an anonymous namespace, so each
// translation unit that includes this header gets its own copy.
#pragma once

#include <cuda.h>
#include <string.h>

#include <mutex>

#include "common.cuh"
#include "w8a8_internal.h"

namespace b200 {
namespace {

constexpr int BM = 128;       // rows per tile = TMEM lanes
constexpr int BK = 128;       // bytes of K per pipeline stage = one swizzle atom
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kSmemBudget = 192 * 1024;          // operand pipeline
constexpr int kStagingPerWarp = 4096;            // epilogue staging block per warp
constexpr int kStagingBytes = kEpilogueWarps * kStagingPerWarp;

// WIDE: the QKV-heads epilogue transposes its table reads and its output through shared
// memory and needs 8 KB per epilogue warp; the operand ring gives up 32 KB for it.
template <int BN, bool WIDE = false>
struct Cfg {
    static constexpr int kABytes = BM * BK;
    static constexpr int kBBytes = BN * BK;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kWarpStaging = WIDE ? 2 * kStagingPerWarp : kStagingPerWarp;
    static constexpr int kStagingTotal = kEpilogueWarps * kWarpStaging;
    static constexpr int kRing = kSmemBudget - (kStagingTotal - kStagingBytes);
    static constexpr int kStages = kRing / kStageBytes > 10 ? 10 : kRing / kStageBytes;
    static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;
    static constexpr int kBarBytes = (2 * kStages + 4) * 8 + 16;
    static constexpr int kSmemBytes = kStages * kStageBytes + kStagingTotal + kBarBytes + 1024;  // + alignment slack
};

struct GemmParams {
    int M, N, K;
    int num_m_blocks, num_n_blocks, num_tiles, num_k_blocks;
    int group_m;     // m-blocks per raster group (keeps a band of A resident in L2)
    int splits, kb_per_split, num_work;  // split-K: work item = (tile, K range); num_work = tiles * splits
    int split_mode;                      // 1 = partials meet in the global workspace, 2 = in cluster shared memory
    int a_stage_bytes;                   // bytes one A load delivers (fewer than 16 KB when M < 128)
    int32_t *ws_partials;                // [splits][M][N] raw partial accumulators (split-K only)
    int *ws_counters;                    // [tiles] arrival tickets, zero between launches
    int b_kx, b_kz;  // W coordinate multipliers: row-major (128,0), slab layout (0,1)
    int a_kx, a_kz;  // the same for A: row-major (128,0), slab-by-slab view (0,1)
    int slabs_per_stage;  // K slabs one copy brings and one pipeline stage holds (1 or 2)
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
    int vec_ok;     // 16-byte vector loads of the per-column vectors / residual are legal
    int tma_store;  // the output can be written through the TMA store path
    int static_weights;  // W may be fetched before the predecessor kernel has completed
    unsigned long long *trace;  // per-CTA timestamps; only read by builds compiled with B200_TRACE
    int *status;                       // where a bounded wait that ran out leaves its code
    unsigned long long wait_limit_ns;  // time limit of every device-side wait of the launch
    int debug_drop_a_load;             // test aid: the producer leaves out its first A tile, so a wait must run out
    // QKV consumer epilogue (OUT == kOutQkvHeads only): head-major fp32 outputs and rotary tables
    float *q_heads, *k_heads, *v_heads;  // [Hq,M,64], [Hkv,M,64], [Hkv,M,64]
    const float *rope_cos, *rope_sin;    // [M,32]
    int n_heads, n_kv_heads;
    float head_eps;
};

// Pseudo output type of the QKV consumer epilogue: per-head RMSNorm + rotary embedding of Q
// and K, plain dequantization of V, all written head-major in fp32.
constexpr int kOutQkvHeads = 4;
constexpr int kHeadDim = 64;

// Per-CTA timestamps for tuning.  Compiled in only with -DB200_TRACE; the shipped library has none.
__device__ __forceinline__ void trace_mark(const GemmParams &p, int slot) {
#ifdef B200_TRACE
    if (p.trace) p.trace[(size_t)blockIdx.x * 16 + slot] = global_timer_ns();
#endif
}

__device__ __forceinline__ void decode_tile(const GemmParams &p, int tile, int &m_blk, int &n_blk);
// Work item -> (tile, split).  The splits of one tile are adjacent so that they run together.
__device__ __forceinline__ void decode_work(const GemmParams &p, int work, int &tile, int &m_blk, int &n_blk,
                                            int &kb0, int &kb1) {
    const int split = work % p.splits;
    tile = work / p.splits;
    decode_tile(p, tile, m_blk, n_blk);
    kb0 = split * p.kb_per_split;
    kb1 = min(p.num_k_blocks, kb0 + p.kb_per_split);
}
__device__ __forceinline__ void decode_tile(const GemmParams &p, int tile, int &m_blk, int &n_blk) {
    const int per_group = p.group_m * p.num_n_blocks;
    const int g = tile / per_group;
    const int r = tile - g * per_group;
    const int gm0 = g * p.group_m;
    const int gsize = min(p.group_m, p.num_m_blocks - gm0);
    n_blk = r / gsize;
    m_blk = gm0 + (r - n_blk * gsize);
}

template <int OUT>
struct OutElem;
template <>
struct OutElem<B200_DT_F16> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __half2 h = __floats2half2_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return __half22float2(*reinterpret_cast<const __half2 *>(&w));
    }
    static __device__ __forceinline__ float load1(const void *p, long long i) {
        return __half2float(reinterpret_cast<const __half *>(p)[i]);
    }
    static __device__ __forceinline__ void store1(void *p, long long i, float v) {
        reinterpret_cast<__half *>(p)[i] = __float2half_rn(v);
    }
};
template <>
struct OutElem<B200_DT_BF16> {
    static __device__ __forceinline__ uint32_t pack(float a, float b) {
        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    static __device__ __forceinline__ float2 unpack(uint32_t w) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(&w));
    }
    static __device__ __forceinline__ float load1(const void *p, long long i) {
        return __bfloat162float(reinterpret_cast<const __nv_bfloat16 *>(p)[i]);
    }
    static __device__ __forceinline__ void store1(void *p, long long i, float v) {
        reinterpret_cast<__nv_bfloat16 *>(p)[i] = __float2bfloat16_rn(v);
    }
};
template <int OUT>
struct Out16 {
    static constexpr int value = (OUT == B200_DT_BF16) ? B200_DT_BF16 : B200_DT_F16;
};

// fp32 epilogue values of 32 consecutive columns of one row from the accumulators in r[]
// (registers, static indexing only).  Vector form: the chunk lies inside N and 16-byte
// accesses to the per-column vectors and the residual are legal.
template <int OUT>
__device__ __forceinline__ void compute32_vec(const GemmParams &p, const uint32_t (&r)[32], int row, bool row_live,
                                              int col0, float row_scale, const uint4 (&res16)[4], float (&v)[32]) {
    {
        const float4 *cs4 = reinterpret_cast<const float4 *>(p.col_scales + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 cs = __ldg(cs4 + g);
            v[4 * g + 0] = dequant_acc((int)r[4 * g + 0], row_scale, cs.x);
            v[4 * g + 1] = dequant_acc((int)r[4 * g + 1], row_scale, cs.y);
            v[4 * g + 2] = dequant_acc((int)r[4 * g + 2], row_scale, cs.z);
            v[4 * g + 3] = dequant_acc((int)r[4 * g + 3], row_scale, cs.w);
        }
    }
    if (p.bias) {
        const float4 *b4 = reinterpret_cast<const float4 *>(p.bias + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 b = __ldg(b4 + g);
            v[4 * g + 0] = __fadd_rn(v[4 * g + 0], b.x);
            v[4 * g + 1] = __fadd_rn(v[4 * g + 1], b.y);
            v[4 * g + 2] = __fadd_rn(v[4 * g + 2], b.z);
            v[4 * g + 3] = __fadd_rn(v[4 * g + 3], b.w);
        }
    }
    if (p.act == B200_ACT_GELU_TANH) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = act_gelu_tanh(v[j]);
    } else if (p.act == B200_ACT_SILU) {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = act_silu(v[j]);
    }
    if (p.gate) {
        const float4 *g4 = reinterpret_cast<const float4 *>(p.gate + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 b = __ldg(g4 + g);
            v[4 * g + 0] = __fmul_rn(v[4 * g + 0], b.x);
            v[4 * g + 1] = __fmul_rn(v[4 * g + 1], b.y);
            v[4 * g + 2] = __fmul_rn(v[4 * g + 2], b.z);
            v[4 * g + 3] = __fmul_rn(v[4 * g + 3], b.w);
        }
    }
    if (p.residual && row_live) {
        if (OUT == B200_DT_F32) {
            const float4 *res = reinterpret_cast<const float4 *>(reinterpret_cast<const float *>(p.residual) +
                                                                 (long long)row * p.ldr + col0);
#pragma unroll
            for (int g = 0; g < 8; ++g) {
                const float4 a = res[g];
                v[4 * g + 0] = __fadd_rn(a.x, v[4 * g + 0]);
                v[4 * g + 1] = __fadd_rn(a.y, v[4 * g + 1]);
                v[4 * g + 2] = __fadd_rn(a.z, v[4 * g + 2]);
                v[4 * g + 3] = __fadd_rn(a.w, v[4 * g + 3]);
            }
        } else {
            constexpr int O = Out16<OUT>::value;
#pragma unroll
            for (int g = 0; g < 4; ++g) {
                const uint4 raw = res16[g];  // fetched one chunk ahead by the caller
                float2 f;
                f = OutElem<O>::unpack(raw.x); v[8 * g + 0] = __fadd_rn(f.x, v[8 * g + 0]); v[8 * g + 1] = __fadd_rn(f.y, v[8 * g + 1]);
                f = OutElem<O>::unpack(raw.y); v[8 * g + 2] = __fadd_rn(f.x, v[8 * g + 2]); v[8 * g + 3] = __fadd_rn(f.y, v[8 * g + 3]);
                f = OutElem<O>::unpack(raw.z); v[8 * g + 4] = __fadd_rn(f.x, v[8 * g + 4]); v[8 * g + 5] = __fadd_rn(f.y, v[8 * g + 5]);
                f = OutElem<O>::unpack(raw.w); v[8 * g + 6] = __fadd_rn(f.x, v[8 * g + 6]); v[8 * g + 7] = __fadd_rn(f.y, v[8 * g + 7]);
            }
        }
    }
}

// Same arithmetic with every per-column access guarded: ragged right edge or unaligned vectors.
template <int OUT>
__device__ __forceinline__ void compute32_guarded(const GemmParams &p, const uint32_t (&r)[32], int row,
                                                  bool row_live, int col0, float row_scale, float (&v)[32]) {
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        float t = 0.0f;
        if (col < p.N) {
            t = dequant_acc((int)r[j], row_scale, p.col_scales[col]);
            if (p.bias) t = __fadd_rn(t, p.bias[col]);
            t = apply_act_rt(t, p.act);
            if (p.gate) t = __fmul_rn(t, p.gate[col]);
            if (p.residual && row_live) {
                const long long ri = (long long)row * p.ldr + col;
                if (OUT == B200_DT_F32) t = __fadd_rn(reinterpret_cast<const float *>(p.residual)[ri], t);
                else t = __fadd_rn(OutElem<Out16<OUT>::value>::load1(p.residual, ri), t);
            }
        }
        v[j] = t;
    }
}

// Direct stores of one row's 32 values (used when the output cannot be described to TMA).
template <int OUT>
__device__ __forceinline__ void store32_direct(const GemmParams &p, const uint32_t (&w)[32], int row, int col0) {
    // w holds 32-bit words: raw accumulators / fp32 bit patterns, or for 16-bit types the 32 values one per word
#pragma unroll
    for (int j = 0; j < 32; ++j) {
        const int col = col0 + j;
        if (col < p.N) {
            const long long oi = (long long)row * p.ldo + col;
            if (OUT == B200_DT_S32 || OUT == B200_DT_F32) reinterpret_cast<uint32_t *>(p.out)[oi] = w[j];
            else OutElem<Out16<OUT>::value>::store1(p.out, oi, __uint_as_float(w[j]));
        }
    }
}

// One 32-row x 32-column block of the output per call and per warp: every thread writes its
// row into a swizzled shared-memory staging block, lane 0 hands the block to the TMA store
// engine, which writes whole row segments and clips at the M / N edges.  A strided per-thread
// store of the same data costs 32 cache-line transactions per instruction instead.
template <int OUT>
__device__ __forceinline__ void stage_and_store(const GemmParams &p, const CUtensorMap *tm_out, uint8_t *stage,
                                                const uint32_t (&w)[32], int lane, int row0, int col0, int seq) {
    constexpr bool k32 = (OUT == B200_DT_S32 || OUT == B200_DT_F32);
    // The warp owns two 2 KB staging blocks of 32 rows x 64 bytes (64-byte swizzle) and alternates
    // between them, so one bulk store can drain while the next block is being filled.  A 16-bit
    // chunk (32 columns) is one block; a 32-bit chunk is two blocks of 16 columns.
    if (k32) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            uint8_t *buf = stage + h * 2048;
            if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
            __syncwarp();
            uint8_t *rowp = buf + lane * 64;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                *reinterpret_cast<uint4 *>(rowp + ((c ^ ((lane >> 1) & 3)) << 4)) =
                    make_uint4(w[16 * h + 4 * c], w[16 * h + 4 * c + 1], w[16 * h + 4 * c + 2], w[16 * h + 4 * c + 3]);
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
                asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(
                                 tm_out),
                             "r"(col0 + 16 * h), "r"(row0), "r"(smem_u32(buf))
                             : "memory");
                asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            }
        }
        return;
    }
    uint8_t *buf = stage + (seq & 1) * 2048;
    if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");
    __syncwarp();
    {
        constexpr int O = Out16<OUT>::value;
        uint8_t *rowp = buf + lane * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4 *>(rowp + ((c ^ ((lane >> 1) & 3)) << 4)) = make_uint4(
                OutElem<O>::pack(__uint_as_float(w[8 * c + 0]), __uint_as_float(w[8 * c + 1])),
                OutElem<O>::pack(__uint_as_float(w[8 * c + 2]), __uint_as_float(w[8 * c + 3])),
                OutElem<O>::pack(__uint_as_float(w[8 * c + 4]), __uint_as_float(w[8 * c + 5])),
                OutElem<O>::pack(__uint_as_float(w[8 * c + 6]), __uint_as_float(w[8 * c + 7])));
    }
    fence_proxy_async_smem();
    __syncwarp();
    if (lane == 0) {
        asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm_out),
                     "r"(col0), "r"(row0), "r"(smem_u32(buf))
                     : "memory");
        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    }
}

// Fetches the 16-bit residual of (row, col0 .. col0+31) into registers; issued one chunk
// ahead of its use so that the L2 round trip hides behind the previous chunk's arithmetic.
template <int OUT>
__device__ __forceinline__ void fetch_residual16(const GemmParams &p, int row, int col0, uint4 (&res16)[4]) {
    if (OUT == B200_DT_S32 || OUT == B200_DT_F32) return;
    if (p.residual && p.vec_ok && row < p.M && col0 + 32 <= p.N) {
        const uint4 *res = reinterpret_cast<const uint4 *>(reinterpret_cast<const uint16_t *>(p.residual) +
                                                           (long long)row * p.ldr + col0);
#pragma unroll
        for (int g = 0; g < 4; ++g) res16[g] = res[g];
    }
}

// GENERAL = false is the lean kernel for the common case (N a multiple of 32, aligned
// buffers): only the vector arithmetic and the TMA store are compiled in, which keeps the
// unrolled epilogue small enough to stay resident in the instruction cache.
template <int OUT, bool GENERAL>
__device__ __forceinline__ void epilogue_chunk(const GemmParams &p, const CUtensorMap *tm_out, uint8_t *stage,
                                               const uint32_t (&r)[32], const uint4 (&res16)[4], int lane, int row0,
                                               int col0, float row_scale, int seq) {
    if (GENERAL && col0 >= p.N) return;  // warp-uniform
    const int row = row0 + lane;
    const bool row_live = row < p.M;
    if (OUT == B200_DT_S32) {
        if (!GENERAL || p.tma_store) stage_and_store<OUT>(p, tm_out, stage, r, lane, row0, col0, seq);
        else if (row_live) store32_direct<OUT>(p, r, row, col0);
        return;
    }
    float v[32];
    if (!GENERAL || (p.vec_ok && col0 + 32 <= p.N)) compute32_vec<OUT>(p, r, row, row_live, col0, row_scale, res16, v);
    else compute32_guarded<OUT>(p, r, row, row_live, col0, row_scale, v);
    uint32_t w[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(v[j]);
    if (!GENERAL || p.tma_store) stage_and_store<OUT>(p, tm_out, stage, w, lane, row0, col0, seq);
    else if (row_live) store32_direct<OUT>(p, w, row, col0);
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
             uint64_t stride2, uint32_t box_rows, uint32_t box_depth = 1) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    cuuint64_t dims[3] = {d0, d1, d2};
    cuuint64_t strides[2] = {stride1, stride2};
    cuuint32_t box[3] = {BK, box_rows, box_depth};
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

// Output matrix [rows, cols] of 16- or 32-bit elements, written in blocks of 32 rows x 64 bytes
// whose shared-memory image uses the swizzle that makes a row-per-thread write conflict-free.
int make_out_map(CUtensorMap *map, const void *base, int dtype, uint64_t cols, uint64_t rows, uint64_t ld) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return fail("cuTensorMapEncodeTiled is not available from this driver");
    const bool k32 = dtype == B200_DT_S32 || dtype == B200_DT_F32;
    const uint64_t esz = k32 ? 4 : 2;
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld * esz};
    cuuint32_t box[2] = {k32 ? 16u : 32u, 32};  // 64-byte rows either way
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, k32 ? CU_TENSOR_MAP_DATA_TYPE_UINT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2,
                    const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail("cuTensorMapEncodeTiled (output) failed (%d)", (int)r);
    return 0;
}

struct DeviceInfo {
    int sms = 0;
    bool attr_set[3][5][4] = {};
    bool pair_attr_set[4] = {};
    bool grouped_attr_set[3] = {};
};
DeviceInfo &device_info(int dev) {
    static DeviceInfo info[64];
    static std::mutex mu;
    std::lock_guard<std::mutex> lock(mu);
    DeviceInfo &d = info[dev & 63];
    if (d.sms == 0) cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
    return d;
}

// Raises a kernel's dynamic shared-memory limit once per device; the per-device flags are only
// read and written under this mutex.
inline std::mutex &attr_mutex() {
    static std::mutex m;
    return m;
}
template <typename Kernel>
int ensure_smem_attr(bool &flag, Kernel kernel, int bytes, const char *what) {
    std::lock_guard<std::mutex> lock(attr_mutex());
    if (flag) return 0;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return fail("cudaFuncSetAttribute(%s, smem=%d): %s", what, bytes, cudaGetErrorString(e));
    flag = true;
    return 0;
}

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline int device_sms() {
    int dev = 0;
    cudaGetDevice(&dev);
    const int sms = device_info(dev).sms;
    return sms > 0 ? sms : 148;
}

}  // namespace
}  // namespace b200
