// A W8A8 linear whose epilogue also produces the NEXT linear's activation codes:
//
//   y[m,:]       = store( residual + gate * act( acc * sx[m] * sw[:] + bias ) )        (as gemm_i8_tcgen05.cu)
//   q[m,:], s[m] = per-row absmax int8 of   y[m, 0:q_cols]                              (plain)
//                                    or of  RMSNorm(y[m, 0:q_cols]) * scale + bias      (rms)
//
// It is the fused form of the reference's call pairs "int8 GEMM + dequant kernel, then the
// quantizer of the next linear": wm_cuda_dequant_gated_residual_f32 / _add_residual_f32 followed
// by wm_cuda_rms_norm_quantize_rows_i8 (src/world_cuda.cu:2088-2120, 2146-2196, 2322-2330 and
// the next layer's :1820-1828), wm_cuda_dequant_silu_quantize_rows_i8
// (src/world_cuda_ops.cu:187-227, call site src/world_cuda.cu:2129-2137), and of the plain
// quantizer wm_cuda_quantize_rows_f32_i8 (src/world_cuda_ops.cu:94-125) applied to a column block
// of the result.  The separate quantizer launch, its read of y and its two reductions disappear.
//
// A row's statistics span q_cols columns = q_cols / 256 column tiles, each owned by a different
// CTA.  Those CTAs form one thread-block cluster (at most 8, so q_cols <= 2048): every CTA keeps
// its 128 x 256 block of results in tensor memory, the per-row partial sums of squares (fp64)
// and partial maxima travel through distributed shared memory to every CTA of the cluster,
// signalled by mbarriers, and each CTA then quantizes its own block.  The maximum is exact in
// any order and the fp64 sum is taken in a fixed order, so codes and scales are bit-identical
// to the stand-alone quantizer run on the stored y.  Column groups beyond the first (the K and
// V blocks of a QKV linear) only run the ordinary epilogue.
//
// Roles per CTA as in the main kernel: warp 0 TMA producer, warp 1 MMA issuer, warps 2-9
// epilogue (two per TMEM sub-partition, 128 columns each); persistent over (row block, column
// group) units, two TMEM accumulators.  Every wait is bounded.
#include "gemm_i8_common.cuh"

namespace b200 {
namespace {

constexpr int RQ_BN = 256;
constexpr int kRqStages = 4;
constexpr int kRqABytes = BM * BK;
constexpr int kRqBBytes = RQ_BN * BK;
constexpr int kRqStageBytes = kRqABytes + kRqBBytes;
constexpr int kRqWarpStaging = 2048;  // one 32-row x 64-byte block per epilogue warp
constexpr int kRqStagingTotal = kEpilogueWarps * kRqWarpStaging;
constexpr int kMaxCluster = 8;
constexpr int kRqSsX = kMaxCluster * BM * 8;  // [source CTA][row] fp64 partial sums of squares
constexpr int kRqMxX = kMaxCluster * BM * 4;  // [source CTA][row] fp32 partial maxima
constexpr int kRqSsHalf = BM * 8;             // hand-over between the two warps that share a row
constexpr int kRqMxHalf = BM * 4;
constexpr int kRqExchange = kRqSsX + kRqMxX + kRqSsHalf + kRqMxHalf;
constexpr int kRqBarBytes = (2 * kRqStages + 4 + 2) * 8 + 16;
constexpr int kRqSmemBytes = kRqStages * kRqStageBytes + kRqStagingTotal + kRqExchange + kRqBarBytes + 1024;
static_assert(kRqSmemBytes <= 227 * 1024, "the row-quantizing GEMM must fit one CTA's shared memory");

struct RowqParams {
    GemmParams g;  // operands, epilogue inputs, launch controls (tile counts are unused here)
    int cs;           // CTAs per cluster = column tiles per quantized row
    int num_groups;   // column groups of cs tiles
    int num_units;    // row blocks x column groups
    int has_out;      // y is stored (through tm_out)
    int q_mode;       // 1 plain, 2 RMSNorm first
    int q_cols;       // cs * 256
    const float *vec_scale;  // RMSNorm gamma / modulation, nullable
    const float *vec_bias;   // nullable
    int scale_is_mod;        // multiply by (1 + vec_scale) instead of vec_scale
    float eps;
    int8_t *q;
    long long ldq;
    float *q_scales;
};

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
        "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void st_shared_cluster_b64(uint32_t addr, double v) {
    asm volatile("st.shared::cluster.b64 [%0], %1;" ::"r"(addr), "l"(__double_as_longlong(v)) : "memory");
}
__device__ __forceinline__ void st_shared_cluster_b32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.b32 [%0], %1;" ::"r"(addr), "r"(__float_as_uint(v)) : "memory");
}

// The two warps that share 32 rows agree on `ok` (a reducing named barrier of 64 threads).
__device__ __forceinline__ bool pair_vote(int bar_id, bool ok) {
    uint32_t both;
    asm volatile(
        "{\n.reg .pred pin, pout;\nsetp.ne.u32 pin, %2, 0;\n"
        "barrier.cta.red.and.pred pout, %1, 64, pin;\nselp.u32 %0, 1, 0, pout;\n}"
        : "=r"(both)
        : "r"(bar_id), "r"((uint32_t)ok)
        : "memory");
    return both != 0;
}
__device__ __forceinline__ void pair_sync(int bar_id) { asm volatile("bar.sync %0, 64;" ::"r"(bar_id) : "memory"); }

// One 32-row x 64-byte block of y through the warp's single staging block and the TMA store
// engine (a 32-column chunk of a 16-bit type, or half a chunk of fp32).
template <int OUT>
__device__ __forceinline__ void rq_store_chunk(const CUtensorMap *tm_out, uint8_t *stage, const uint32_t (&w)[32],
                                               int lane, int row0, int col0) {
    constexpr bool k32 = OUT == B200_DT_F32;
#pragma unroll
    for (int h = 0; h < (k32 ? 2 : 1); ++h) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
        uint8_t *rowp = stage + lane * 64;
#pragma unroll
        for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4 *>(rowp + ((c ^ ((lane >> 1) & 3)) << 4)) =
                make_uint4(w[16 * h + 4 * c], w[16 * h + 4 * c + 1], w[16 * h + 4 * c + 2], w[16 * h + 4 * c + 3]);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm_out),
                         "r"(col0 + 16 * h), "r"(row0), "r"(smem_u32(stage))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}

// RMSNorm tail on 32 consecutive columns of one row: t = x * inv_rms [* scale] [+ bias].
__device__ __forceinline__ void normalize32(const RowqParams &rp, float (&v)[32], int col0, float inv) {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = __fmul_rn(v[j], inv);
    if (rp.vec_scale) {
        const float4 *s4 = reinterpret_cast<const float4 *>(rp.vec_scale + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            float4 s = __ldg(s4 + g);
            if (rp.scale_is_mod) {
                s.x = __fadd_rn(1.0f, s.x); s.y = __fadd_rn(1.0f, s.y);
                s.z = __fadd_rn(1.0f, s.z); s.w = __fadd_rn(1.0f, s.w);
            }
            v[4 * g + 0] = __fmul_rn(v[4 * g + 0], s.x);
            v[4 * g + 1] = __fmul_rn(v[4 * g + 1], s.y);
            v[4 * g + 2] = __fmul_rn(v[4 * g + 2], s.z);
            v[4 * g + 3] = __fmul_rn(v[4 * g + 3], s.w);
        }
    }
    if (rp.vec_bias) {
        const float4 *b4 = reinterpret_cast<const float4 *>(rp.vec_bias + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 b = __ldg(b4 + g);
            v[4 * g + 0] = __fadd_rn(v[4 * g + 0], b.x);
            v[4 * g + 1] = __fadd_rn(v[4 * g + 1], b.y);
            v[4 * g + 2] = __fadd_rn(v[4 * g + 2], b.z);
            v[4 * g + 3] = __fadd_rn(v[4 * g + 3], b.w);
        }
    }
}

template <int OUT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_i8_rowq_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                        const __grid_constant__ CUtensorMap tm_out, const RowqParams rp) {
    const GemmParams &p = rp.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + kRqStages * kRqStageBytes;
    double *ss_x = reinterpret_cast<double *>(staging + kRqStagingTotal);
    float *mx_x = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ss_x) + kRqSsX);
    double *ss_half = reinterpret_cast<double *>(reinterpret_cast<uint8_t *>(mx_x) + kRqMxX);
    float *mx_half = reinterpret_cast<float *>(reinterpret_cast<uint8_t *>(ss_half) + kRqSsHalf);
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(reinterpret_cast<uint8_t *>(mx_half) + kRqMxHalf);
    uint64_t *bar_empty = bar_full + kRqStages;
    uint64_t *bar_tfull = bar_empty + kRqStages;
    uint64_t *bar_tempty = bar_tfull + 2;
    uint64_t *bar_x = bar_tempty + 2;  // [0] sums of squares have arrived, [1] maxima have arrived
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_x + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int cs = rp.cs;
    const uint32_t rank = cluster_cta_rank();
    const int cluster_id = blockIdx.x / cs;
    const int num_clusters = gridDim.x / cs;

    pdl_trigger();
    if (threadIdx.x == 0) {
        trace_mark(p, 0);
        for (int s = 0; s < kRqStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_tfull[b], 1);
            mbar_init(&bar_tempty[b], kEpilogueWarps);
            mbar_init(&bar_x[b], (uint32_t)(cs * 4));  // one arrival per sending warp of every CTA of the cluster
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (rp.has_out) tma_prefetch_desc(&tm_out);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 2 * RQ_BN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // every CTA's barriers exist before any CTA signals them
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) trace_mark(p, 1);

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            bool first = true;
            // weights nothing in the stream writes: the first ring of W tiles goes out before the
            // predecessor kernel (whose output is our A operand) has finished
            int prefetched = 0;
            if (p.static_weights && cluster_id < rp.num_units) {
                const int grp = cluster_id % rp.num_groups;
                const int n0 = (grp * cs + (int)rank) * RQ_BN;
                if (n0 < p.N) {
                    prefetched = min(p.num_k_blocks, kRqStages);
                    for (int i = 0; i < prefetched; ++i) {
                        uint8_t *sa = smem + i * kRqStageBytes;
                        mbar_arrive_expect_tx(&bar_full[i], (uint32_t)(p.a_stage_bytes + kRqBBytes));
                        tma_load_3d(sa + kRqABytes, &tm_b, &bar_full[i], i * p.b_kx, n0, i * p.b_kz);
                    }
                }
            }
            pdl_wait();
            for (int u = cluster_id; ok && u < rp.num_units; u += num_clusters) {
                const int m0 = (u / rp.num_groups) * BM;
                const int n0 = ((u % rp.num_groups) * cs + (int)rank) * RQ_BN;
                if (n0 >= p.N) continue;
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    uint8_t *sa = smem + s * kRqStageBytes;
                    const bool drop = p.debug_drop_a_load && first && kb == 0;
                    if (prefetched > 0) {
                        --prefetched;
                        if (!drop) tma_load_3d(sa, &tm_a, &bar_full[s], kb * BK, m0, 0);
                    } else {
                        ok = mbar_wait_bounded(&bar_empty[s], ph ^ 1u, wctx, KS_TIMEOUT_SMEM_EMPTY);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&bar_full[s], (uint32_t)(p.a_stage_bytes + kRqBBytes));
                        if (!drop) tma_load_3d(sa, &tm_a, &bar_full[s], kb * BK, m0, 0);
                        tma_load_3d(sa + kRqABytes, &tm_b, &bar_full[s], kb * p.b_kx, n0, kb * p.b_kz);
                    }
                    if (++s == kRqStages) { s = 0; ph ^= 1u; }
                }
                first = false;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(BM, RQ_BN);
            int s = 0, t = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int u = cluster_id; ok && u < rp.num_units; u += num_clusters) {
                const int n0 = ((u % rp.num_groups) * cs + (int)rank) * RQ_BN;
                if (n0 >= p.N) continue;
                const int b = t & 1;
                const uint32_t tph = (uint32_t)(t >> 1) & 1u;
                ok = mbar_wait_bounded(&bar_tempty[b], tph ^ 1u, wctx, KS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * RQ_BN);
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    ok = mbar_wait_bounded(&bar_full[s], ph, wctx, KS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    if (t == 0 && kb == 0) trace_mark(p, 2);
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * kRqStageBytes);
                    const uint64_t da = umma_smem_desc_k128(sa);
                    const uint64_t db = umma_smem_desc_k128(sa + kRqABytes);
#pragma unroll
                    for (int j = 0; j < BK / 32; ++j)
                        umma_i8(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (uint32_t)((kb | j) != 0));
                    umma_commit(&bar_empty[s]);
                    if (++s == kRqStages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(&bar_tfull[b]);
                if (t == 0) trace_mark(p, 3);
                ++t;
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const int sub = warp & 3;   // TMEM sub-partition = 32 rows of the tile
        const int half = ew >> 2;   // which 128 of the tile's 256 columns
        const int trow = sub * 32 + lane;  // this thread's row within the tile
        const int vote_bar = 2 + sub;
        uint8_t *stage = staging + ew * kRqWarpStaging;
        const bool rms = rp.q_mode == 2;
        pdl_wait();
        int t = 0;
        uint32_t qi = 0;  // quantized units finished so far: phase of the exchange barriers
        bool carry_ok = true;
        for (int u = cluster_id; u < rp.num_units; u += num_clusters) {
            const int m_blk = u / rp.num_groups, grp = u % rp.num_groups;
            const int n0 = (grp * cs + (int)rank) * RQ_BN;
            if (n0 >= p.N) continue;
            const int b = t & 1;
            const uint32_t tph = (uint32_t)(t >> 1) & 1u;
            const int row0 = m_blk * BM + sub * 32;
            const int row = row0 + lane;
            const bool row_live = row < p.M;
            const int colbase = n0 + half * (RQ_BN / 2);
            {
                const int line_col = colbase + lane * 32;
                if (lane < 4 && line_col < p.N) {
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(p.col_scales + line_col));
                    if (p.bias) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.bias + line_col));
                    if (p.gate) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gate + line_col));
                }
            }
            const float row_scale = row_live ? __ldg(p.row_scales + row) : 0.0f;
            uint4 res[4];
            fetch_residual16<OUT>(p, row, colbase, res);
            bool ok = mbar_wait_bounded(&bar_tfull[b], tph, wctx, KS_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok && carry_ok);
            ok = pair_vote(vote_bar, ok);  // the two warps of a sub-partition go on together or not at all
            if (!ok) break;
            const bool tr = warp == 2 && lane == 0 && t == 0;
            if (tr) trace_mark(p, 4);
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(b * RQ_BN + half * (RQ_BN / 2));
            const bool quant = grp == 0;
            const bool store_y = rp.has_out && row0 < p.M;

            // ---- pass 1: the ordinary epilogue; the values to be quantized go back into tensor memory
            double ss = 0.0;
            float amax = 0.0f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                const int col0 = colbase + c * 32;
                if (col0 >= p.N) break;  // ragged last column group (never a quantized one); warp-uniform
                uint32_t r[32];
                tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                tmem_ld_wait();
                float v[32];
                compute32_vec<OUT>(p, r, row, row_live, col0, row_scale, res, v);
                if (c < 3) fetch_residual16<OUT>(p, row, col0 + 32, res);
                uint32_t w[32];
                if (OUT == B200_DT_F32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(v[j]);
                } else {
                    // what is stored is what gets normalised and quantized: round first
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        w[j] = OutElem<Out16<OUT>::value>::pack(v[2 * j], v[2 * j + 1]);
                        const float2 f = OutElem<Out16<OUT>::value>::unpack(w[j]);
                        v[2 * j] = f.x;
                        v[2 * j + 1] = f.y;
                    }
                }
                if (quant) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(v[j]);
                    tmem_st_32x32(taddr + (uint32_t)(c * 32), r);
                    if (rms) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) ss = fma((double)v[j], (double)v[j], ss);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
                    }
                }
                if (store_y) rq_store_chunk<OUT>(&tm_out, stage, w, lane, row0, col0);
            }
            if (!quant) {
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_tempty[b]);
                ++t;
                continue;
            }
            tmem_st_wait();
            if (tr) trace_mark(p, 5);
            const uint32_t xph = qi & 1u;
            bool okx = true;
            float inv = 1.0f;
            if (rms) {
                // ---- exchange 1: sums of squares of all cs column tiles of the row
                if (half == 1) ss_half[trow] = ss;
                pair_sync(vote_bar);
                if (half == 0) {
                    ss += ss_half[trow];
                    const uint32_t slot = smem_u32(&ss_x[rank * BM + trow]);
                    for (int dst = 0; dst < cs; ++dst) st_shared_cluster_b64(cluster_map_shared(slot, (uint32_t)dst), ss);
                    __syncwarp();
                    if (lane == 0)
                        for (int dst = 0; dst < cs; ++dst)
                            mbar_arrive_cluster(cluster_map_shared(smem_u32(&bar_x[0]), (uint32_t)dst));
                }
                okx = mbar_wait_bounded_cluster(&bar_x[0], xph, wctx, KS_TIMEOUT_ROW_EXCHANGE);
                okx = __all_sync(0xffffffffu, okx);
                if (tr) trace_mark(p, 6);
                double tot = 0.0;
                for (int s = 0; s < cs; ++s) tot += ss_x[s * BM + trow];  // fixed order: identical in every CTA
                inv = (float)(1.0 / sqrt(tot / (double)rp.q_cols + (double)rp.eps));
                // ---- pass 2: maximum of the normalised values
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    normalize32(rp, v, colbase + c * 32, inv);
#pragma unroll
                    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
                }
            }
            // ---- exchange 2: row maxima.  Without the first exchange in between, a fast CTA could write
            // the next unit's maxima while a slow one still reads this unit's: two buffers alternate then.
            if (tr) trace_mark(p, 7);
            float *mx_buf = (rms || xph == 0) ? mx_x : reinterpret_cast<float *>(ss_x);
            if (half == 1) mx_half[trow] = amax;
            okx = pair_vote(vote_bar, okx);
            if (okx) {
                if (half == 0) {
                    amax = fmaxf(amax, mx_half[trow]);
                    const uint32_t slot = smem_u32(&mx_buf[rank * BM + trow]);
                    for (int dst = 0; dst < cs; ++dst) st_shared_cluster_b32(cluster_map_shared(slot, (uint32_t)dst), amax);
                    __syncwarp();
                    if (lane == 0)
                        for (int dst = 0; dst < cs; ++dst)
                            mbar_arrive_cluster(cluster_map_shared(smem_u32(&bar_x[1]), (uint32_t)dst));
                }
                okx = mbar_wait_bounded_cluster(&bar_x[1], xph, wctx, KS_TIMEOUT_ROW_EXCHANGE);
                okx = __all_sync(0xffffffffu, okx);
            }
            if (tr) trace_mark(p, 8);
            if (okx) {
                float m = 0.0f;
                for (int s = 0; s < cs; ++s) m = fmaxf(m, mx_buf[s * BM + trow]);
                const RowScale scale = make_row_scale(m);
                if (rank == 0 && half == 0 && row_live) rp.q_scales[row] = scale.scale;
                // ---- pass 3: codes
                int8_t *qrow = rp.q + (long long)row * rp.ldq + colbase;
#pragma unroll 1
                for (int c = 0; c < 4; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                    tmem_ld_wait();
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
                    if (rms) normalize32(rp, v, colbase + c * 32, inv);
                    uint32_t codes[8];
#pragma unroll
                    for (int g = 0; g < 8; ++g)
                        codes[g] = pack_biased4(quantize_biased(v[4 * g], scale), quantize_biased(v[4 * g + 1], scale),
                                                quantize_biased(v[4 * g + 2], scale), quantize_biased(v[4 * g + 3], scale));
                    if (row_live) {
                        uint4 *dst = reinterpret_cast<uint4 *>(qrow + c * 32);
                        dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
                        dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
                    }
                }
            }
            if (tr) trace_mark(p, 9);
            carry_ok = okx;
            ++qi;
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_tempty[b]);
            ++t;
        }
        // the staging block must outlive the bulk store that reads it
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    __syncthreads();
    if (*abort_flag) {
        // a wait ran out somewhere: give copies and MMAs already in flight time to land
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) trace_mark(p, 10);
    tc_fence_before_sync();
    cluster_sync_all();  // no CTA exits while another may still write its shared memory or signal its barriers
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * RQ_BN);
    }
}

struct RowqDeviceInfo {
    bool attr_set[3] = {};
    int max_clusters[3][kMaxCluster + 1] = {};
};
RowqDeviceInfo &rowq_device_info(int dev) {
    static RowqDeviceInfo info[64];
    return info[dev & 63];
}

template <int OUT>
int launch_rowq(const LinearArgs &a, RowqParams &rp, cudaStream_t stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    RowqDeviceInfo &di = rowq_device_info(dev);
    constexpr int oi = OUT == B200_DT_F32 ? 0 : (OUT == B200_DT_F16 ? 1 : 2);
    if (ensure_smem_attr(di.attr_set[oi], gemm_i8_rowq_kernel<OUT>, kRqSmemBytes, "gemm_i8_rowq_kernel")) return 1;
    GemmParams &p = rp.g;
    const int a_rows = a.m >= BM ? BM : ((a.m + 15) / 16) * 16;
    p.a_stage_bytes = a_rows * BK;
    p.num_k_blocks = (a.k + BK - 1) / BK;
    CUtensorMap tm_a, tm_b, tm_out;
    if (make_map(&tm_a, a.x, (uint64_t)a.k, (uint64_t)a.m, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.m,
                 (uint32_t)a_rows))
        return 1;
    if (a.w_layout == B200_W_SLAB128) {
        if (make_map(&tm_b, a.w, BK, (uint64_t)a.n, (uint64_t)(a.k / BK), BK, (uint64_t)a.n * BK, RQ_BN)) return 1;
        p.b_kx = 0;
        p.b_kz = 1;
    } else {
        if (make_map(&tm_b, a.w, (uint64_t)a.k, (uint64_t)a.n, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.n, RQ_BN))
            return 1;
        p.b_kx = BK;
        p.b_kz = 0;
    }
    memset(&tm_out, 0, sizeof(tm_out));
    if (rp.has_out && make_out_map(&tm_out, a.out, a.out_dtype, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldo)) return 1;

    // how many clusters of this size the device can hold at once (asked once per device and size)
    int max_clusters = 0;
    {
        std::lock_guard<std::mutex> lock(attr_mutex());
        max_clusters = di.max_clusters[oi][rp.cs];
        if (max_clusters == 0) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)(rp.cs * 64));
            cfg.blockDim = dim3(kThreads);
            cfg.dynamicSmemBytes = kRqSmemBytes;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = (unsigned)rp.cs;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_i8_rowq_kernel<OUT>, &cfg) != cudaSuccess || n <= 0) {
                cudaGetLastError();
                n = device_sms() / rp.cs;  // fall back to "as many as fit by count"
                if (n <= 0) n = 1;
            }
            max_clusters = di.max_clusters[oi][rp.cs] = n;
        }
    }
    const int clusters = rp.num_units < max_clusters ? rp.num_units : max_clusters;
    cudaError_t le = launch_kernel_cluster(gemm_i8_rowq_kernel<OUT>, dim3((unsigned)(clusters * rp.cs)), dim3(kThreads),
                                           (size_t)kRqSmemBytes, stream, (unsigned)rp.cs, tm_a, tm_b, tm_out, rp);
    if (le != cudaSuccess) return fail("launching gemm_i8_rowq: %s", cudaGetErrorString(le));
    return check_launch("gemm_i8_rowq");
}

}  // namespace

const char *linear_requant_unsupported(const LinearArgs &a, const RowQuantSpec &qs) {
    if (qs.mode != B200_RQ_PLAIN && qs.mode != B200_RQ_RMS) return "unknown row-quantizer mode";
    if (!qs.q || !qs.scales) return "q and q_scales are required";
    if (qs.cols <= 0 || qs.cols % RQ_BN != 0 || qs.cols / RQ_BN > kMaxCluster) return "q_cols must be a multiple of 256, at most 2048";
    if (qs.cols > a.n) return "q_cols exceeds N";
    if (a.n % 32 != 0) return "N must be a multiple of 32";
    if (qs.ldq < qs.cols || qs.ldq % 16 != 0 || !aligned16(qs.q)) return "q must be 16-byte aligned with a row stride that is a multiple of 16";
    if (a.out_dtype != B200_DT_F32 && a.out_dtype != B200_DT_F16 && a.out_dtype != B200_DT_BF16) return "y must be fp32, fp16 or bf16";
    const size_t esz = a.out_dtype == B200_DT_F32 ? 4 : 2;
    if (a.out && (!aligned16(a.out) || (a.ldo * esz) % 16 != 0)) return "y must be 16-byte aligned with 16-byte aligned rows";
    if (a.residual && (!aligned16(a.residual) || (a.ldr * esz) % 16 != 0)) return "the residual must be 16-byte aligned with 16-byte aligned rows";
    if (!aligned16(a.col_scales) || (a.bias && !aligned16(a.bias)) || (a.gate && !aligned16(a.gate))) return "per-column vectors must be 16-byte aligned";
    if ((qs.vec_scale && !aligned16(qs.vec_scale)) || (qs.vec_bias && !aligned16(qs.vec_bias))) return "norm vectors must be 16-byte aligned";
    return nullptr;
}

int linear_requant(const LinearArgs &a_in, const RowQuantSpec &qs, cudaStream_t stream) {
    LinearArgs a = a_in;
    if (!a.out) {  // codes only: the shared argument check wants a plausible output description
        a.out = qs.q;
        a.ldo = a.n;
    }
    if (gemm_can_implement(a, true)) return 1;
    if (a.out_dtype == B200_DT_S32) return fail("linear_requant writes fp32, fp16 or bf16");
    if (const char *why = linear_requant_unsupported(a_in, qs)) {
        // Rows wider than a cluster holds (the MLP hidden: 32 column tiles) or buffers the fused form cannot
        // take: with y stored, the same result comes from the linear followed by the stand-alone quantizer
        // reading y -- two launches, identical codes (the fused kernel quantizes what it stores, too).
        const bool shape_ok = qs.q && qs.scales && qs.cols > 0 && qs.cols <= a.n && qs.ldq >= qs.cols &&
                              (qs.mode == B200_RQ_PLAIN || qs.mode == B200_RQ_RMS);
        if (!a_in.out || !shape_ok)
            return fail("linear_requant M=%d K=%d N=%d q_cols=%d cannot run fused: %s; the two-launch form needs y "
                        "and valid q / q_scales", a.m, a.k, a.n, qs.cols, why);
        if (gemm_launch(a_in, nullptr, 0, stream)) return 1;
        if (qs.mode == B200_RQ_PLAIN)
            return quantize_rows(a_in.out, a.out_dtype, a.ldo, qs.q, qs.ldq, qs.scales, a.m, qs.cols, stream);
        return rms_norm_quantize_rows(a_in.out, a.out_dtype, a.ldo, qs.vec_scale, qs.scale_is_mod, qs.vec_bias, qs.q,
                                      qs.ldq, qs.scales, a.m, qs.cols, qs.eps, stream);
    }
    RowqParams rp{};
    GemmParams &p = rp.g;
    p.M = a.m; p.N = a.n; p.K = a.k;
    p.row_scales = a.row_scales; p.col_scales = a.col_scales; p.bias = a.bias; p.gate = a.gate;
    p.residual = a.residual; p.ldr = a.ldr; p.out = a_in.out; p.ldo = a.ldo;
    p.out_dtype = a.out_dtype; p.act = a.act;
    p.vec_ok = 1;
    p.tma_store = 1;
    p.static_weights = a.static_weights;
    p.trace = gemm_trace_buffer();
    p.status = status_slot(true);
    p.wait_limit_ns = wait_limit_ns();
    p.debug_drop_a_load = take_debug_drop();
    rp.cs = qs.cols / RQ_BN;
    const int tiles_n = (a.n + RQ_BN - 1) / RQ_BN;
    rp.num_groups = (tiles_n + rp.cs - 1) / rp.cs;
    rp.num_units = ((a.m + BM - 1) / BM) * rp.num_groups;
    rp.has_out = a_in.out != nullptr;
    rp.q_mode = qs.mode;
    rp.q_cols = qs.cols;
    rp.vec_scale = qs.mode == B200_RQ_RMS ? qs.vec_scale : nullptr;
    rp.vec_bias = qs.mode == B200_RQ_RMS ? qs.vec_bias : nullptr;
    rp.scale_is_mod = qs.scale_is_mod;
    rp.eps = qs.eps;
    rp.q = qs.q; rp.ldq = qs.ldq; rp.q_scales = qs.scales;
    switch (a.out_dtype) {
        case B200_DT_F32: return launch_rowq<B200_DT_F32>(a, rp, stream);
        case B200_DT_F16: return launch_rowq<B200_DT_F16>(a, rp, stream);
        default: return launch_rowq<B200_DT_BF16>(a, rp, stream);
    }
}

}  // namespace b200
