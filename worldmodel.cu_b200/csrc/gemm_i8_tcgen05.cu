// s8 x s8 -> s32 GEMM for sm_100a with the epilogue of a W8A8 linear fused in.
//
//   acc[m,n] = sum_k x[m,k] * w[n,k]          x: int8 [M,K] row-major, w: int8 [N,K]
//   y[m,n]   = residual + gate * act(acc * sx[m] * sw[n] + bias[n])      (optional parts)
//
// It replaces the reference's CUTLASS Ampere-class mma.sync instantiation and the
// separate dequant kernels that re-read its int32 scratch
// (src/world_cuda_ops.cu:529-599, 229-262).
//
// Structure: a persistent kernel, one CTA per SM, 320 threads in three roles.
//   warp 0    : TMA producer.  Streams 128-row x 128-byte operand slabs of A and W into a
//               ring of shared-memory stages (128-byte swizzle), signalling `full` mbarriers.
//   warp 1    : MMA issuer.  One thread issues tcgen05.mma (kind i8, 128 x BN x 32 per
//               instruction, four per stage) into one of two TMEM accumulators and commits
//               completion to the stage's `empty` barrier / the accumulator's `full` barrier.
//   warps 2-9 : epilogue.  Two warps per 32-lane TMEM sub-partition (= 32 rows of the tile),
//               each taking half of the tile's columns: they pull accumulators out with
//               tcgen05.ld (double-buffered in registers), apply the fused epilogue and
//               store.  The second accumulator lets tile i+1's main loop run under tile
//               i's epilogue.
// Both operands are K-major in memory already, so nothing is transposed; the operand
// descriptors only differ in height.  Every wait is bounded (see mbar_wait_bounded): on
// expiry the CTA drains and the kernel leaves a status word instead of hanging.
//
// Roofline: tensor-bound for M >= ~1024 (2*M*N*K ops), HBM-bound on the N*K weight bytes
// for M <= 128.
#include <atomic>

#include "gemm_i8_common.cuh"

namespace b200 {

// Built-in split-K scratch for callers that cannot allocate device memory (see
// linear_static_scratch below).  It lives in the module's global segment: every GPU that
// loads the library holds these bytes until the process exits.  Zero-initialized at load;
// the split-K kernel returns its ticket counters to zero, so it is ready again after each call.
constexpr size_t kStaticScratchBytes = 4096 + (size_t)8 * 1024 * 1024;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

namespace {

// (tile configuration, parameter block, epilogue arithmetic and tensor-map helpers: gemm_i8_common.cuh)

// QKV consumer as a GEMM epilogue: one thread holds one token's 64 accumulators of one head
// (two 32-column TMEM loads), so the per-head sum of squares needs no shuffle.  Q and K heads
// are normalised by 1/sqrt(mean(z^2) + eps) (fp64 sum) and rotated with the token's cos/sin
// row: out[p] = a*c - b*s, out[32+p] = b*c + a*s for the interleaved pair (a, b) =
// (z[2p], z[2p+1]); V heads are only dequantized.
//
// A row per thread is the worst global access pattern (32 lines per instruction), so both
// directions go through shared memory with a 16-byte XOR swizzle that is conflict-free for
// the row-per-thread side and for the coalesced side:
//   tables  [32 rows][8 x 16 B] of cos and of sin, loaded coalesced once per tile by the two
//           warps that share the 32 rows (one loads cos, the other sin);
//   output  a head's 32 rows x 256 B are contiguous in the head-major result; they leave in
//           two passes of 32 rows x 128 B, written row-per-thread, read back 4 rows per
//           instruction and stored as full 128-byte lines.
__device__ __forceinline__ uint32_t swz16(int row, int chunk) { return (uint32_t)(row * 128 + ((chunk ^ (row & 7)) << 4)); }

__device__ __forceinline__ void qkv_store_pass(uint8_t *out_stage, float *head_base, int row0, int lane, int M,
                                               int byte_off) {
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = 4 * i + (lane >> 3), c = lane & 7;
        const float4 val = *reinterpret_cast<const float4 *>(out_stage + swz16(r, c));
        if (row0 + r < M)
            *reinterpret_cast<float4 *>(reinterpret_cast<uint8_t *>(head_base + (long long)(row0 + r) * kHeadDim) +
                                        byte_off + c * 16) = val;
    }
    __syncwarp();  // the block is free again
}

__device__ __forceinline__ void qkv_head_epilogue(const GemmParams &p, uint32_t taddr, const uint8_t *cos_tab,
                                                  const uint8_t *sin_tab, uint8_t *out_stage, int row0, int lane,
                                                  int head, float row_scale) {
    uint32_t ra[32], rb[32];
    tmem_ld_32x32(taddr, ra);
    tmem_ld_32x32(taddr + 32u, rb);
    tmem_ld_wait();
    const int col0 = head * kHeadDim;
    float z[kHeadDim];
    {
        const float4 *cs4 = reinterpret_cast<const float4 *>(p.col_scales + col0);
#pragma unroll
        for (int g = 0; g < 8; ++g) {
            const float4 ca = __ldg(cs4 + g), cb = __ldg(cs4 + 8 + g);
            z[4 * g + 0] = dequant_acc((int)ra[4 * g + 0], row_scale, ca.x);
            z[4 * g + 1] = dequant_acc((int)ra[4 * g + 1], row_scale, ca.y);
            z[4 * g + 2] = dequant_acc((int)ra[4 * g + 2], row_scale, ca.z);
            z[4 * g + 3] = dequant_acc((int)ra[4 * g + 3], row_scale, ca.w);
            z[32 + 4 * g + 0] = dequant_acc((int)rb[4 * g + 0], row_scale, cb.x);
            z[32 + 4 * g + 1] = dequant_acc((int)rb[4 * g + 1], row_scale, cb.y);
            z[32 + 4 * g + 2] = dequant_acc((int)rb[4 * g + 2], row_scale, cb.z);
            z[32 + 4 * g + 3] = dequant_acc((int)rb[4 * g + 3], row_scale, cb.w);
        }
    }
    if (p.bias) {
        const float4 *b4 = reinterpret_cast<const float4 *>(p.bias + col0);
#pragma unroll
        for (int g = 0; g < 16; ++g) {
            const float4 b = __ldg(b4 + g);
            z[4 * g + 0] = __fadd_rn(z[4 * g + 0], b.x);
            z[4 * g + 1] = __fadd_rn(z[4 * g + 1], b.y);
            z[4 * g + 2] = __fadd_rn(z[4 * g + 2], b.z);
            z[4 * g + 3] = __fadd_rn(z[4 * g + 3], b.w);
        }
    }
    const int qk_heads = p.n_heads + p.n_kv_heads;
    if (head >= qk_heads) {  // V: dequantized only (warp-uniform branch)
        float *base = p.v_heads + (long long)(head - qk_heads) * p.M * kHeadDim;
#pragma unroll
        for (int pass = 0; pass < 2; ++pass) {
#pragma unroll
            for (int g = 0; g < 8; ++g)
                *reinterpret_cast<float4 *>(out_stage + swz16(lane, g)) =
                    make_float4(z[32 * pass + 4 * g], z[32 * pass + 4 * g + 1], z[32 * pass + 4 * g + 2],
                                z[32 * pass + 4 * g + 3]);
            qkv_store_pass(out_stage, base, row0, lane, p.M, pass * 128);
        }
        return;
    }
    double s0 = 0.0, s1 = 0.0, s2 = 0.0, s3 = 0.0;  // four chains: fp64 latency, not order, is the concern
#pragma unroll
    for (int j = 0; j < kHeadDim; j += 4) {
        s0 = fma((double)z[j], (double)z[j], s0);
        s1 = fma((double)z[j + 1], (double)z[j + 1], s1);
        s2 = fma((double)z[j + 2], (double)z[j + 2], s2);
        s3 = fma((double)z[j + 3], (double)z[j + 3], s3);
    }
    const double ss = (s0 + s1) + (s2 + s3);
    const float inv = (float)(1.0 / sqrt(ss / (double)kHeadDim + (double)p.head_eps));
    float *base = head < p.n_heads ? p.q_heads + (long long)head * p.M * kHeadDim
                                   : p.k_heads + (long long)(head - p.n_heads) * p.M * kHeadDim;
    // pass 0: out[0..31] = a*c - b*s; pass 1: out[32..63] = b*c + a*s
#pragma unroll
    for (int g = 0; g < 8; ++g) {
        const float4 c = *reinterpret_cast<const float4 *>(cos_tab + swz16(lane, g));
        const float4 sn = *reinterpret_cast<const float4 *>(sin_tab + swz16(lane, g));
        const float a0 = __fmul_rn(z[8 * g + 0], inv), b0 = __fmul_rn(z[8 * g + 1], inv);
        const float a1 = __fmul_rn(z[8 * g + 2], inv), b1 = __fmul_rn(z[8 * g + 3], inv);
        const float a2 = __fmul_rn(z[8 * g + 4], inv), b2 = __fmul_rn(z[8 * g + 5], inv);
        const float a3 = __fmul_rn(z[8 * g + 6], inv), b3 = __fmul_rn(z[8 * g + 7], inv);
        *reinterpret_cast<float4 *>(out_stage + swz16(lane, g)) =
            make_float4(__fsub_rn(__fmul_rn(a0, c.x), __fmul_rn(b0, sn.x)),
                        __fsub_rn(__fmul_rn(a1, c.y), __fmul_rn(b1, sn.y)),
                        __fsub_rn(__fmul_rn(a2, c.z), __fmul_rn(b2, sn.z)),
                        __fsub_rn(__fmul_rn(a3, c.w), __fmul_rn(b3, sn.w)));
        // the second half is kept in z (its inputs are consumed) until the first pass has left
        z[8 * g + 0] = __fadd_rn(__fmul_rn(b0, c.x), __fmul_rn(a0, sn.x));
        z[8 * g + 1] = __fadd_rn(__fmul_rn(b1, c.y), __fmul_rn(a1, sn.y));
        z[8 * g + 2] = __fadd_rn(__fmul_rn(b2, c.z), __fmul_rn(a2, sn.z));
        z[8 * g + 3] = __fadd_rn(__fmul_rn(b3, c.w), __fmul_rn(a3, sn.w));
    }
    qkv_store_pass(out_stage, base, row0, lane, p.M, 0);
#pragma unroll
    for (int g = 0; g < 8; ++g)
        *reinterpret_cast<float4 *>(out_stage + swz16(lane, g)) =
            make_float4(z[8 * g + 0], z[8 * g + 1], z[8 * g + 2], z[8 * g + 3]);
    qkv_store_pass(out_stage, base, row0, lane, p.M, 128);
}

// SPLITK: 0 = one CTA owns the whole K range of a tile; 1 = K split over CTAs that meet in a
// global workspace; 2 = K split over the CTAs of a cluster that meet in shared memory.
template <int BN, int OUT, bool GENERAL, int SPLITK>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_i8_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                   const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
    using C = Cfg<BN, OUT == kOutQkvHeads>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + C::kStages * C::kStageBytes;  // 1024-byte aligned: stage sizes are multiples of 1 KB
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(staging + C::kStagingTotal);
    uint64_t *bar_empty = bar_full + C::kStages;
    uint64_t *bar_tfull = bar_empty + C::kStages;
    uint64_t *bar_tempty = bar_tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_tempty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile int *last_flag = abort_flag + 1;  // split-K: "this CTA holds the last partial of the tile"
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Slabs of K per pipeline stage: 1, or 2 for narrow tiles, where the copy engine's cost per copy (not per
    // byte) bounds the main loop: one copy then brings two 128-byte slabs of A (or of W), the ring has half as
    // many stages of twice the size, and a stage feeds eight MMAs instead of four.
    const int kd = p.slabs_per_stage;
    const int n_stages = C::kStages / kd;
    const int stage_bytes = kd * C::kStageBytes;
    const int b_off = kd * C::kABytes;  // the W slabs of a stage follow its A slabs

    pdl_trigger();  // the next kernel of the stream may be scheduled from here on
    if (threadIdx.x == 0) {
        trace_mark(p, 0);
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_tfull[b], 1);
            mbar_init(&bar_tempty[b], kEpilogueWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (p.tma_store) tma_prefetch_desc(&tm_out);
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
            trace_mark(p, 1);
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            // Weights that nothing in the stream writes can be requested before the predecessor
            // kernel has finished: the first ring of W tiles is put in flight, then the thread
            // waits for the predecessor (whose output is our A operand) and adds the A tiles.
            int prefetched = 0;
            if (p.static_weights && blockIdx.x < p.num_work) {
                int tile, m_blk, n_blk, kb0, kb1;
                decode_work(p, blockIdx.x, tile, m_blk, n_blk, kb0, kb1);
                prefetched = min((kb1 - kb0) / kd, n_stages);
                for (int i = 0; i < prefetched; ++i) {
                    uint8_t *sa = smem + i * stage_bytes;
                    mbar_arrive_expect_tx(&bar_full[i], (uint32_t)(kd * (p.a_stage_bytes + C::kBBytes)));
                    tma_load_3d(sa + b_off, &tm_b, &bar_full[i], (kb0 + i * kd) * p.b_kx, n_blk * BN,
                                (kb0 + i * kd) * p.b_kz);
                }
            }
            pdl_wait();
            for (int work = blockIdx.x; ok && work < p.num_work; work += gridDim.x) {
                int tile, m_blk, n_blk, kb0, kb1;
                decode_work(p, work, tile, m_blk, n_blk, kb0, kb1);
                const int m0 = m_blk * BM, n0 = n_blk * BN;
                for (int kb = kb0; kb < kb1; kb += kd) {
                    uint8_t *sa = smem + s * stage_bytes;
                    // test aid: leaving out the very first A tile makes the MMA issuer's wait run out
                    const bool drop = p.debug_drop_a_load && work == (int)blockIdx.x && kb == kb0;
                    if (prefetched > 0) {
                        // stage already armed and its W tile already requested
                        --prefetched;
                        if (!drop) tma_load_3d(sa, &tm_a, &bar_full[s], kb * p.a_kx, m0, kb * p.a_kz);
                    } else {
                        ok = mbar_wait_bounded(&bar_empty[s], ph ^ 1u, wctx,
                                               KS_TIMEOUT_SMEM_EMPTY);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&bar_full[s], (uint32_t)(kd * (p.a_stage_bytes + C::kBBytes)));
                        if (!drop) tma_load_3d(sa, &tm_a, &bar_full[s], kb * p.a_kx, m0, kb * p.a_kz);
                        tma_load_3d(sa + b_off, &tm_b, &bar_full[s], kb * p.b_kx, n0, kb * p.b_kz);
                    }
                    if (++s == n_stages) { s = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();  // the whole warp must reach the closing barrier together
        if (SPLITK == 2) {
            cluster_sync_all();
            cluster_sync_all();
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(BM, BN);
            int s = 0;
            uint32_t ph = 0;
            int t = 0;
            bool ok = true;
            for (int work = blockIdx.x; ok && work < p.num_work; work += gridDim.x, ++t) {
                int tile, m_blk, n_blk, kb0, kb1;
                decode_work(p, work, tile, m_blk, n_blk, kb0, kb1);
                const int b = t & 1;
                const uint32_t tph = (uint32_t)(t >> 1) & 1u;
                ok = mbar_wait_bounded(&bar_tempty[b], tph ^ 1u, wctx, KS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
                for (int kb = kb0; kb < kb1; kb += kd) {
                    ok = mbar_wait_bounded(&bar_full[s], ph, wctx, KS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    if (t == 0 && kb == kb0) trace_mark(p, 2);
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * stage_bytes);
                    for (int d = 0; d < kd; ++d) {
                        const uint64_t da = umma_smem_desc_k128(sa + (uint32_t)(d * p.a_stage_bytes));
                        const uint64_t db = umma_smem_desc_k128(sa + (uint32_t)(b_off + d * C::kBBytes));
#pragma unroll
                        for (int j = 0; j < BK / 32; ++j)
                            umma_i8(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc,
                                    (uint32_t)(((kb - kb0) | d | j) != 0));
                    }
                    umma_commit(&bar_empty[s]);
                    if (++s == n_stages) { s = 0; ph ^= 1u; }
                }
                if (ok) umma_commit(&bar_tfull[b]);
                trace_mark(p, 3);
            }
        }
        __syncwarp();
        if (SPLITK == 2) {
            cluster_sync_all();
            cluster_sync_all();
        }
    } else {
        // Eight epilogue warps: two per TMEM sub-partition, each taking half of the columns,
        // so every SM sub-core has two warps to hide latencies with.
        const int ew = warp - 2;
        const int sub = warp & 3;          // TMEM sub-partition this warp may read
        const int half = ew >> 2;          // which half of the tile's columns
        constexpr int kCols = BN / 2;      // columns per warp
        constexpr int kChunks = kCols / 32;
        uint8_t *stage = staging + ew * C::kWarpStaging;
        pdl_wait();  // before the first read of the scales / residual and the first write of the output
        int t = 0;
        int seq = 0;  // running count of this warp's staged stores: alternates the 16-bit staging halves
        bool ok = true;
        for (int work = blockIdx.x; ok && work < p.num_work; work += gridDim.x, ++t) {
            int tile, m_blk, n_blk, kb0, kb1;
            decode_work(p, work, tile, m_blk, n_blk, kb0, kb1);
            const int b = t & 1;
            const uint32_t tph = (uint32_t)(t >> 1) & 1u;
            // Before the accumulator is ready: pull this warp's slice of the per-column vectors
            // into L1, and fetch the row scale and the first residual chunk.
            const int row0 = m_blk * BM + sub * 32;
            const int colbase = n_blk * BN + half * kCols;
            float row_scale = 0.0f;
            uint4 res_a[4], res_b[4];
            if (OUT != B200_DT_S32) {
                const int line_col = colbase + lane * 32;  // one 128-byte line of fp32 per lane
                if (lane * 32 < kCols && line_col < p.N) {
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(p.col_scales + line_col));
                    if (p.bias) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.bias + line_col));
                    if (p.gate) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gate + line_col));
                }
                if (row0 + lane < p.M) row_scale = __ldg(p.row_scales + row0 + lane);
                fetch_residual16<OUT>(p, row0 + lane, colbase, res_a);
                if (OUT == kOutQkvHeads) {  // this warp's rotary table (cos or sin) of the 32 rows, coalesced
                    const float *tab = half ? p.rope_sin : p.rope_cos;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int r = 4 * i + (lane >> 3), c = lane & 7;
                        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (row0 + r < p.M)
                            val = __ldg(reinterpret_cast<const float4 *>(tab + (long long)(row0 + r) * (kHeadDim / 2)) + c);
                        *reinterpret_cast<float4 *>(stage + swz16(r, c)) = val;
                    }
                }
            }
            ok = mbar_wait_bounded(&bar_tfull[b], tph, wctx, KS_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (SPLITK == 1) {
                // the eight warps meet at named barriers below: they go on together or not at all
                uint32_t all;
                asm volatile(
                    "{\n.reg .pred pin, pout;\nsetp.ne.u32 pin, %1, 0;\n"
                    "barrier.cta.red.and.pred pout, 1, %2, pin;\nselp.u32 %0, 1, 0, pout;\n}"
                    : "=r"(all)
                    : "r"((uint32_t)ok), "n"(kEpilogueWarps * 32)
                    : "memory");
                ok = all != 0;
            }
            // (in a cluster every thread still has to meet the cluster barriers; the QKV-heads
            // epilogue first lets the two warps that share a table agree on the outcome)
            if (!ok && SPLITK != 2 && OUT != kOutQkvHeads) break;
            if (warp == 2 && lane == 0) trace_mark(p, 4);
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(b * BN + half * kCols);
            if (SPLITK == 2) {
                // Split-K inside a cluster: the `splits` CTAs of a cluster hold partial sums of the
                // same tile.  CTA r reduces and finishes the column slice [r, r+1) * BN / splits:
                // every CTA pushes the other slices of its partial into their owner's shared memory
                // (the operand ring, idle by now), one cluster barrier later every owner adds what
                // it received to its own accumulators and runs the fused epilogue.  No global
                // scratch, no atomics; integer sums are exact in any order.
                const uint32_t rank = cluster_cta_rank();
                const int slice_cols = BN / p.splits;        // 32, 64 or 128
                const int own_chunks = slice_cols / 32;
                const uint32_t ring = smem_u32(smem);
                cluster_sync_all();  // every CTA of the cluster has finished reading its operand ring
                if (warp == 2 && lane == 0) trace_mark(p, 8);
                if (ok && row0 < p.M) {  // a sub-partition whose 32 rows all lie beyond M has nothing to send
#pragma unroll 1
                    for (int c = 0; c < kChunks; ++c) {
                        const int col_in_tile = half * kCols + c * 32;
                        const uint32_t owner = (uint32_t)(col_in_tile / slice_cols);
                        if (owner == rank) continue;
                        uint32_t r[32];
                        tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                        tmem_ld_wait();
                        const uint32_t slot = rank < owner ? rank : rank - 1u;
                        const int j = (col_in_tile - (int)owner * slice_cols) / 32;  // chunk within the owner's slice
                        // Receive layout [slot][sub-partition][chunk][vector g][lane]: one store
                        // instruction of the warp fills 512 contiguous bytes, and the owner's warp
                        // of the same sub-partition reads them back lane for lane.
                        const uint32_t off =
                            (uint32_t)((((slot * 4 + sub) * own_chunks + j) * 8) * 512 + lane * 16);
                        const uint32_t remote = cluster_map_shared(ring + off, owner);
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            st_shared_cluster_v4(remote + (uint32_t)(g * 512), r[4 * g], r[4 * g + 1], r[4 * g + 2],
                                                 r[4 * g + 3]);
                    }
                }
                if (warp == 2 && lane == 0) trace_mark(p, 9);
                cluster_sync_all();  // all partial slices have landed in their owners
                if (warp == 2 && lane == 0) trace_mark(p, 10);
                if (ok && row0 < p.M) {
#pragma unroll 1
                    for (int j = half; j < own_chunks; j += 2) {
                        const int col_in_tile = (int)rank * slice_cols + j * 32;
                        uint32_t r[32];
                        tmem_ld_32x32(tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(b * BN + col_in_tile), r);
                        tmem_ld_wait();
                        for (int slot = 0; slot < p.splits - 1; ++slot) {
                            const uint8_t *src = smem + (((slot * 4 + sub) * own_chunks + j) * 8) * 512 + lane * 16;
#pragma unroll
                            for (int g = 0; g < 8; ++g) {
                                const uint4 q = *reinterpret_cast<const uint4 *>(src + g * 512);
                                r[4 * g + 0] += q.x;
                                r[4 * g + 1] += q.y;
                                r[4 * g + 2] += q.z;
                                r[4 * g + 3] += q.w;
                            }
                        }
                        const int col0 = n_blk * BN + col_in_tile;
                        uint4 res[4];
                        fetch_residual16<OUT>(p, row0 + lane, col0, res);
                        epilogue_chunk<OUT, true>(p, &tm_out, stage, r, res, lane, row0, col0, row_scale, seq++);
                    }
                }
                if (warp == 2 && lane == 0) trace_mark(p, 5);
                break;  // a clustered launch gives every CTA exactly one work item
            }
            if (SPLITK == 1) {
                // Split-K: this CTA holds one of `splits` partial sums of the tile.  Every CTA
                // parks its raw int32 partial in the workspace and takes a ticket; the CTA that
                // draws the last ticket adds the partials (integer sums: exact in any order)
                // and runs the fused epilogue.  Nobody waits for anybody.
                const int split = work % p.splits;
                const int row = row0 + lane;
                int32_t *mine = p.ws_partials + ((long long)split * p.M + row) * p.N;
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                    tmem_ld_wait();
                    const int col0 = colbase + c * 32;
                    if (row < p.M) {
#pragma unroll
                        for (int g = 0; g < 8; ++g)
                            if (col0 + 4 * g < p.N)
                                __stcg(reinterpret_cast<int4 *>(mine + col0) + g,
                                       make_int4((int)r[4 * g], (int)r[4 * g + 1], (int)r[4 * g + 2], (int)r[4 * g + 3]));
                    }
                }
                __threadfence();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_tempty[b]);  // this warp has drained its accumulator slice
                asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueWarps * 32) : "memory");
                if (ew == 0 && lane == 0) {
                    const int old = atomicAdd(p.ws_counters + tile, 1);
                    const int last = old == p.splits - 1;
                    if (last) p.ws_counters[tile] = 0;  // leave the ticket counter clean for the next launch
                    *last_flag = last;
                }
                asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueWarps * 32) : "memory");
                if (*last_flag) {
                    __threadfence();
#pragma unroll 1
                    for (int c = 0; c < kChunks; ++c) {
                        const int col0 = colbase + c * 32;
                        if (col0 >= p.N) break;
                        uint32_t r[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) r[j] = 0u;
                        if (row < p.M) {
                            for (int sp = 0; sp < p.splits; ++sp) {
                                const int4 *src = reinterpret_cast<const int4 *>(
                                    p.ws_partials + ((long long)sp * p.M + row) * p.N + col0);
#pragma unroll
                                for (int g = 0; g < 8; ++g) {
                                    if (col0 + 4 * g < p.N) {
                                        const int4 q = __ldcg(src + g);
                                        r[4 * g + 0] += (uint32_t)q.x;
                                        r[4 * g + 1] += (uint32_t)q.y;
                                        r[4 * g + 2] += (uint32_t)q.z;
                                        r[4 * g + 3] += (uint32_t)q.w;
                                    }
                                }
                            }
                        }
                        uint4 res[4];
                        fetch_residual16<OUT>(p, row, col0, res);
                        epilogue_chunk<OUT, true>(p, &tm_out, stage, r, res, lane, row0, col0, row_scale, seq++);
                    }
                }
                if (warp == 2 && lane == 0) trace_mark(p, 5);
                continue;
            }
            if constexpr (OUT == kOutQkvHeads) {
                // The two warps of a sub-partition share the 32 rows: the first 4 KB of the lower
                // warp's staging holds the cos rows, of the upper warp's the sin rows; each warp's
                // second 4 KB is its own output block.  (The tables were loaded before the wait.)
                const uint8_t *cos_tab = staging + (ew & 3) * C::kWarpStaging;  // warps ew and ew + 4 share `sub`
                const uint8_t *sin_tab = staging + (4 + (ew & 3)) * C::kWarpStaging;
                {  // both tables are in place, and both warps saw the accumulator arrive (or neither goes on)
                    uint32_t both;
                    asm volatile(
                        "{\n.reg .pred pin, pout;\nsetp.ne.u32 pin, %2, 0;\n"
                        "barrier.cta.red.and.pred pout, %1, 64, pin;\nselp.u32 %0, 1, 0, pout;\n}"
                        : "=r"(both)
                        : "r"(2 + sub), "r"((uint32_t)ok)
                        : "memory");
                    ok = both != 0;
                    if (!ok) break;
                }
#pragma unroll 1
                for (int hh = 0; hh < kCols / kHeadDim; ++hh) {
                    const int col0 = colbase + hh * kHeadDim;
                    if (col0 >= p.N) break;  // warp-uniform: N is a whole number of heads
                    qkv_head_epilogue(p, taddr + (uint32_t)(hh * kHeadDim), cos_tab, sin_tab, stage + kStagingPerWarp,
                                      row0, lane, col0 / kHeadDim, row_scale);
                }
                asm volatile("bar.sync %0, 64;" ::"r"(2 + sub) : "memory");  // both warps are done with the tables
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar_tempty[b]);
                if (warp == 2 && lane == 0) trace_mark(p, 5);
                continue;
            }
            // two register buffers: the TMEM load (and residual fetch) of chunk c+1 is in flight
            // while chunk c is processed
            uint32_t ra[32], rb[32];
            tmem_ld_32x32(taddr, ra);
#pragma unroll
            for (int c = 0; c < kChunks; c += 2) {
                tmem_ld_wait();
                if (c + 1 < kChunks) {
                    tmem_ld_32x32(taddr + (uint32_t)((c + 1) * 32), rb);
                    fetch_residual16<OUT>(p, row0 + lane, colbase + (c + 1) * 32, res_b);
                }
                epilogue_chunk<OUT, GENERAL>(p, &tm_out, stage, ra, res_a, lane, row0, colbase + c * 32, row_scale, seq++);
                if (c + 1 < kChunks) {
                    tmem_ld_wait();
                    if (c + 2 < kChunks) {
                        tmem_ld_32x32(taddr + (uint32_t)((c + 2) * 32), ra);
                        fetch_residual16<OUT>(p, row0 + lane, colbase + (c + 2) * 32, res_a);
                    }
                    epilogue_chunk<OUT, GENERAL>(p, &tm_out, stage, rb, res_b, lane, row0, colbase + (c + 1) * 32, row_scale,
                                        seq++);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_tempty[b]);
            if (warp == 2 && lane == 0) trace_mark(p, 5);
        }
        // the staging blocks must outlive the bulk stores that read them
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    __syncthreads();
    if (threadIdx.x == 0) trace_mark(p, 6);
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

// ---------------------------------------------------------------- CTA-pair kernel (M >= 256)
// The same GEMM with two CTAs of a cluster working on one 256 x 256 tile.  Each CTA loads
// its own 128 rows of A and only HALF of the tile's W rows (128 of 256) per K slab: 32 KB
// instead of 48 KB per CTA for the same amount of tensor work.  The L2 -> SM operand feed is
// what bounds the single-CTA kernel at large M (about 15 TB/s aggregate on B200), so a third
// less traffic is a third more throughput there.  The leader CTA (cluster rank 0) issues
// tcgen05.mma.cta_group::2, which reads both CTAs' shared memory and writes both CTAs'
// tensor memory.  Barrier wiring:
//   full[s]   lives in the leader; both CTAs' TMA loads count their bytes on it;
//   empty[s]  one in each CTA; the leader's commit signals both;
//   tfull[b]  one in each CTA; the leader's commit signals both;
//   tempty[b] lives in the leader; the epilogue warps of both CTAs arrive on it.
// No CTA leaves before a closing cluster barrier, so no signal ever targets a CTA that has exited.
constexpr int kPairStageBytes = 2 * BM * BK;  // 16 KB of A + 16 KB of W per CTA and stage
constexpr int kPairStages = kSmemBudget / kPairStageBytes;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + kStagingBytes + (2 * kPairStages + 4) * 8 + 16 + 1024;

template <int OUT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_i8_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                        const __grid_constant__ CUtensorMap tm_out, const GemmParams p) {
    constexpr int BN = 256;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + kPairStages * kPairStageBytes;
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(staging + kStagingBytes);
    uint64_t *bar_empty = bar_full + kPairStages;
    uint64_t *bar_tfull = bar_empty + kPairStages;
    uint64_t *bar_tempty = bar_tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_tempty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta_rank = cluster_cta_rank();  // 0 = leader
    const int pair_id = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    // K slabs per stage: with 2, one copy per operand brings a box two slabs deep (half the copies for the same
    // bytes in flight: three stages of 64 KB instead of six of 32 KB); a stage then feeds eight MMAs.
    const int kd = p.slabs_per_stage;
    const int n_stages = kPairStages / kd;
    const int stage_bytes = kd * kPairStageBytes;
    const int b_off = kd * BM * BK;  // the W slabs of a stage follow its A slabs

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kPairStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_tfull[b], 1);
            mbar_init(&bar_tempty[b], 2 * kEpilogueWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        tma_prefetch_desc(&tm_out);
    }
    if (warp == 1) {
        tmem_alloc_pair(tmem_slot, 512);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();  // both CTAs' barriers exist before either signals the other
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t ph = 0;
            bool ok = true;
            // Weights that nothing in the stream writes: the W tiles of the first ring are requested before the
            // predecessor kernel (whose output is the A operand) has finished; the A tiles follow after the wait.
            int prefetched = 0;
            if (p.static_weights && pair_id < p.num_tiles) {
                int m_blk, n_blk;
                decode_tile(p, pair_id, m_blk, n_blk);
                const int n0 = n_blk * BN + (int)cta_rank * (BN / 2);
                prefetched = min(p.num_k_blocks / kd, n_stages);
                for (int i = 0; i < prefetched; ++i) {
                    const uint32_t full_in_leader = cluster_map_shared(smem_u32(&bar_full[i]), 0);
                    if (cta_rank == 0) mbar_arrive_expect_tx(&bar_full[i], 2u * (uint32_t)stage_bytes);
                    tma_load_3d_pair(smem + i * stage_bytes + b_off, &tm_b, full_in_leader, (i * kd) * p.b_kx, n0,
                                     (i * kd) * p.b_kz);
                }
            }
            pdl_wait();
            for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs) {
                int m_blk, n_blk;
                decode_tile(p, tile, m_blk, n_blk);
                const int m0 = m_blk * 2 * BM + (int)cta_rank * BM;
                const int n0 = n_blk * BN + (int)cta_rank * (BN / 2);
                for (int kb = 0; kb < p.num_k_blocks; kb += kd) {
                    uint8_t *sa = smem + s * stage_bytes;
                    const uint32_t full_in_leader = cluster_map_shared(smem_u32(&bar_full[s]), 0);
                    if (prefetched > 0) {
                        --prefetched;  // stage already armed, its W tile already requested
                        tma_load_3d_pair(sa, &tm_a, full_in_leader, kb * p.a_kx, m0, kb * p.a_kz);
                    } else {
                        ok = mbar_wait_bounded(&bar_empty[s], ph ^ 1u, wctx, KS_TIMEOUT_SMEM_EMPTY);
                        if (!ok) break;
                        if (cta_rank == 0) mbar_arrive_expect_tx(&bar_full[s], 2u * (uint32_t)stage_bytes);  // both CTAs' bytes
                        tma_load_3d_pair(sa, &tm_a, full_in_leader, kb * p.a_kx, m0, kb * p.a_kz);
                        tma_load_3d_pair(sa + b_off, &tm_b, full_in_leader, kb * p.b_kx, n0, kb * p.b_kz);
                    }
                    if (++s == n_stages) { s = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0 && cta_rank == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(2 * BM, BN);
            int s = 0;
            uint32_t ph = 0;
            int t = 0;
            bool ok = true;
            for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++t) {
                const int b = t & 1;
                const uint32_t tph = (uint32_t)(t >> 1) & 1u;
                ok = mbar_wait_bounded(&bar_tempty[b], tph ^ 1u, wctx, KS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < p.num_k_blocks; kb += kd) {
                    ok = mbar_wait_bounded(&bar_full[s], ph, wctx, KS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * stage_bytes);
                    for (int d = 0; d < kd; ++d) {
                        const uint64_t da = umma_smem_desc_k128(sa + (uint32_t)(d * BM * BK));
                        const uint64_t db = umma_smem_desc_k128(sa + (uint32_t)(b_off + d * BM * BK));
#pragma unroll
                        for (int j = 0; j < BK / 32; ++j)
                            umma_i8_pair(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc,
                                         (uint32_t)((kb | d | j) != 0));
                    }
                    umma_commit_pair(smem_u32(&bar_empty[s]));                         // my own stage is free
                    umma_commit_pair(cluster_map_shared(smem_u32(&bar_empty[s]), 1));  // and the peer's
                    if (++s == n_stages) { s = 0; ph ^= 1u; }
                }
                if (ok) {
                    umma_commit_pair(smem_u32(&bar_tfull[b]));
                    umma_commit_pair(cluster_map_shared(smem_u32(&bar_tfull[b]), 1));
                }
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const int sub = warp & 3;
        const int half = ew >> 2;
        constexpr int kCols = BN / 2;
        constexpr int kChunks = kCols / 32;
        uint8_t *stage = staging + ew * kStagingPerWarp;
        pdl_wait();
        int t = 0;
        int seq = 0;
        bool ok = true;
        for (int tile = pair_id; ok && tile < p.num_tiles; tile += num_pairs, ++t) {
            int m_blk, n_blk;
            decode_tile(p, tile, m_blk, n_blk);
            const int b = t & 1;
            const uint32_t tph = (uint32_t)(t >> 1) & 1u;
            const int row0 = m_blk * 2 * BM + (int)cta_rank * BM + sub * 32;
            const int colbase = n_blk * BN + half * kCols;
            float row_scale = 0.0f;
            uint4 res_a[4], res_b[4];
            if (OUT != B200_DT_S32) {
                const int line_col = colbase + lane * 32;
                if (lane * 32 < kCols && line_col < p.N) {
                    asm volatile("prefetch.global.L1 [%0];" ::"l"(p.col_scales + line_col));
                    if (p.bias) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.bias + line_col));
                    if (p.gate) asm volatile("prefetch.global.L1 [%0];" ::"l"(p.gate + line_col));
                }
                if (row0 + lane < p.M) row_scale = __ldg(p.row_scales + row0 + lane);
                fetch_residual16<OUT>(p, row0 + lane, colbase, res_a);
            }
            ok = mbar_wait_bounded(&bar_tfull[b], tph, wctx, KS_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(b * BN + half * kCols);
            uint32_t ra[32], rb[32];
            tmem_ld_32x32(taddr, ra);
#pragma unroll
            for (int c = 0; c < kChunks; c += 2) {
                tmem_ld_wait();
                if (c + 1 < kChunks) {
                    tmem_ld_32x32(taddr + (uint32_t)((c + 1) * 32), rb);
                    fetch_residual16<OUT>(p, row0 + lane, colbase + (c + 1) * 32, res_b);
                }
                if (colbase + c * 32 < p.N && row0 < p.M)
                    epilogue_chunk<OUT, false>(p, &tm_out, stage, ra, res_a, lane, row0, colbase + c * 32, row_scale,
                                               seq++);
                if (c + 1 < kChunks) {
                    tmem_ld_wait();
                    if (c + 2 < kChunks) {
                        tmem_ld_32x32(taddr + (uint32_t)((c + 2) * 32), ra);
                        fetch_residual16<OUT>(p, row0 + lane, colbase + (c + 2) * 32, res_a);
                    }
                    if (colbase + (c + 1) * 32 < p.N && row0 < p.M)
                        epilogue_chunk<OUT, false>(p, &tm_out, stage, rb, res_b, lane, row0, colbase + (c + 1) * 32,
                                                   row_scale, seq++);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_cluster(cluster_map_shared(smem_u32(&bar_tempty[b]), 0));
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    __syncthreads();
    if (*abort_flag) {
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
    }
    tc_fence_before_sync();
    cluster_sync_all();  // nobody frees tensor memory or exits while the other CTA may still signal it
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc_pair(tmem_base, 512);
    }
}

// ---------------------------------------------------------------- grouped skinny linears (M <= 128)
// Many independent weight-bound linears in ONE launch.  A single skinny linear cannot use the
// memory system: its few megabytes of weights stream in well under a microsecond, but launch,
// first-byte latency, epilogue and hand-over cost four to five.  Here the persistent CTAs walk
// the 128 x 256 tiles of ALL problems in one sequence, so the operand ring never drains between
// problems and the weights of problem g+1 are already in flight while the tiles of problem g are
// being finished.  Every problem has a single block of rows (M <= 128); its A rows are loaded as
// they are (ceil16(M) rows), the MMA spans 128 lanes and the lanes beyond M are never read back.
// Problem descriptors and the two tensor maps of each problem travel in kernel-parameter space.
// 72 x (3 tensor maps of 128 bytes + a 64-byte record) + a 40-byte header = 32 296 of the 32 764 bytes a
// kernel may take as parameters.
constexpr int kMaxGroup = 72;
struct GroupedProblem {
    const float *row_scales, *col_scales, *bias;
    const void *residual;
    void *out;
    int ldo, ldr;   // row strides in elements (below 2^31)
    int m, n;
    int tile0;      // index of the problem's first tile in the launch-wide sequence
    unsigned short k_blocks;  // K slabs of 128 bytes (K <= 8 388 480)
    unsigned char vec_ok;     // 16-byte vector access to the per-column vectors / residual is legal
    unsigned char tma_store;  // the output is aligned for bulk-tensor stores (else plain stores)
};
static_assert(sizeof(GroupedProblem) == 64, "the grouped problem record is sized to fit 72 per launch");
struct GroupedParams {
    CUtensorMap tm_a[kMaxGroup];
    CUtensorMap tm_w[kMaxGroup];
    CUtensorMap tm_out[kMaxGroup];
    GroupedProblem prob[kMaxGroup];
    int count, total_tiles, act, out_dtype, w_kx, w_kz;
    int static_weights;  // W may be fetched before the predecessor kernel has completed
    int *status;
    unsigned long long wait_limit_ns;
};

template <int OUT>
__global__ void __launch_bounds__(kThreads, 1) gemm_i8_grouped_kernel(const __grid_constant__ GroupedParams gp) {
    constexpr int BN = 256;
    using C = Cfg<BN>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + C::kStages * C::kStageBytes;
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(staging + C::kStagingTotal);
    uint64_t *bar_empty = bar_full + C::kStages;
    uint64_t *bar_tfull = bar_empty + C::kStages;
    uint64_t *bar_tempty = bar_tfull + 2;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_tempty + 2);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const WaitCtx wctx{abort_flag, gp.status, gp.wait_limit_ns};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&bar_tfull[b], 1);
            mbar_init(&bar_tempty[b], kEpilogueWarps);
        }
        *abort_flag = 0;
        fence_mbar_init();
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
            int s = 0, g = 0;
            uint32_t ph = 0;
            bool ok = true;
            // weights nothing in the stream writes: the first ring of W tiles of this CTA's first tile goes out
            // before the predecessor kernel has finished; the A tiles follow once it has
            int prefetched = 0;
            if (gp.static_weights && (int)blockIdx.x < gp.total_tiles) {
                int g0 = 0;
                while (g0 + 1 < gp.count && (int)blockIdx.x >= gp.prob[g0 + 1].tile0) ++g0;
                const GroupedProblem &q = gp.prob[g0];
                const int n0 = ((int)blockIdx.x - q.tile0) * BN;
                prefetched = min((int)q.k_blocks, C::kStages);
                for (int i = 0; i < prefetched; ++i) {
                    uint8_t *sa = smem + i * C::kStageBytes;
                    mbar_arrive_expect_tx(&bar_full[i], (uint32_t)(((q.m + 15) / 16) * 16 * BK + C::kBBytes));
                    tma_load_3d(sa + C::kABytes, &gp.tm_w[g0], &bar_full[i], i * gp.w_kx, n0, i * gp.w_kz);
                }
            }
            pdl_wait();
            for (int work = blockIdx.x; ok && work < gp.total_tiles; work += gridDim.x) {
                while (g + 1 < gp.count && work >= gp.prob[g + 1].tile0) ++g;  // tiles are visited in order
                const GroupedProblem &q = gp.prob[g];
                const int n0 = (work - q.tile0) * BN;
                for (int kb = 0; kb < q.k_blocks; ++kb) {
                    uint8_t *sa = smem + s * C::kStageBytes;
                    if (prefetched > 0) {  // stage already armed, its W tile already requested
                        --prefetched;
                        tma_load_3d(sa, &gp.tm_a[g], &bar_full[s], kb * BK, 0, 0);
                    } else {
                        ok = mbar_wait_bounded(&bar_empty[s], ph ^ 1u, wctx, KS_TIMEOUT_SMEM_EMPTY);
                        if (!ok) break;
                        mbar_arrive_expect_tx(&bar_full[s], (uint32_t)(((q.m + 15) / 16) * 16 * BK + C::kBBytes));
                        tma_load_3d(sa, &gp.tm_a[g], &bar_full[s], kb * BK, 0, 0);
                        tma_load_3d(sa + C::kABytes, &gp.tm_w[g], &bar_full[s], kb * gp.w_kx, n0, kb * gp.w_kz);
                    }
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(BM, BN);
            int s = 0, g = 0, t = 0;
            uint32_t ph = 0;
            bool ok = true;
            for (int work = blockIdx.x; ok && work < gp.total_tiles; work += gridDim.x, ++t) {
                while (g + 1 < gp.count && work >= gp.prob[g + 1].tile0) ++g;
                const int k_blocks = gp.prob[g].k_blocks;
                const int b = t & 1;
                const uint32_t tph = (uint32_t)(t >> 1) & 1u;
                ok = mbar_wait_bounded(&bar_tempty[b], tph ^ 1u, wctx, KS_TIMEOUT_TMEM_EMPTY);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + (uint32_t)(b * BN);
                for (int kb = 0; kb < k_blocks; ++kb) {
                    ok = mbar_wait_bounded(&bar_full[s], ph, wctx, KS_TIMEOUT_SMEM_FULL);
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
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const int sub = warp & 3;
        const int half = ew >> 2;
        constexpr int kCols = BN / 2;
        constexpr int kChunks = kCols / 32;
        uint8_t *stage = staging + ew * C::kWarpStaging;
        pdl_wait();
        int t = 0, g = 0, seq = 0;
        bool ok = true;
        for (int work = blockIdx.x; ok && work < gp.total_tiles; work += gridDim.x, ++t) {
            while (g + 1 < gp.count && work >= gp.prob[g + 1].tile0) ++g;
            const GroupedProblem &q = gp.prob[g];
            // the shared epilogue code takes the single-problem parameter block: fill in what it reads
            GemmParams p{};
            p.M = q.m; p.N = q.n;
            p.row_scales = q.row_scales; p.col_scales = q.col_scales; p.bias = q.bias; p.gate = nullptr;
            p.residual = q.residual; p.ldr = q.ldr; p.out = q.out; p.ldo = q.ldo;
            p.out_dtype = gp.out_dtype; p.act = gp.act; p.vec_ok = q.vec_ok; p.tma_store = q.tma_store;
            const int b = t & 1;
            const uint32_t tph = (uint32_t)(t >> 1) & 1u;
            const int row0 = sub * 32;
            const int colbase = (work - q.tile0) * BN + half * kCols;
            float row_scale = 0.0f;
            if (row0 + lane < p.M) row_scale = __ldg(p.row_scales + row0 + lane);
            ok = mbar_wait_bounded(&bar_tfull[b], tph, wctx, KS_TIMEOUT_TMEM_FULL);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            if (row0 < p.M) {  // a sub-partition whose 32 lanes all lie beyond M has nothing to write
                const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + (uint32_t)(b * BN + half * kCols);
#pragma unroll 1
                for (int c = 0; c < kChunks; ++c) {
                    const int col0 = colbase + c * 32;
                    if (col0 >= p.N) break;
                    uint32_t r[32];
                    uint4 res[4];
                    tmem_ld_32x32(taddr + (uint32_t)(c * 32), r);
                    fetch_residual16<OUT>(p, row0 + lane, col0, res);
                    tmem_ld_wait();
                    epilogue_chunk<OUT, true>(p, &gp.tm_out[g], stage, r, res, lane, row0, col0, row_scale, seq++);
                }
            }
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar_tempty[b]);
        }
        // the staging blocks must outlive the bulk stores that read them
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    __syncthreads();
    if (*abort_flag) {
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


std::atomic<int> g_one_slab_stages{0};  // tuning: 1 = never put two K slabs into one pipeline stage

template <int BN, int OUT, bool GENERAL, int SPLITK>
int launch_bn_g(const LinearArgs &a, GemmParams &p, int slot, cudaStream_t stream) {
    using C = Cfg<BN, OUT == kOutQkvHeads>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    DeviceInfo &di = device_info(dev);
    constexpr int kVariant = SPLITK == 2 ? 3 : (SPLITK == 1 ? 2 : (GENERAL ? 1 : 0));
    if (ensure_smem_attr(di.attr_set[slot][OUT][kVariant], gemm_i8_kernel<BN, OUT, GENERAL, SPLITK>, C::kSmemBytes,
                         "gemm_i8_kernel"))
        return 1;
    p.num_m_blocks = (a.m + BM - 1) / BM;
    p.num_n_blocks = (a.n + BN - 1) / BN;
    p.num_tiles = p.num_m_blocks * p.num_n_blocks;
    p.num_k_blocks = (a.k + BK - 1) / BK;
    p.group_m = 32;
    if (p.splits < 1) p.splits = 1;
    p.kb_per_split = (p.num_k_blocks + p.splits - 1) / p.splits;
    p.num_work = p.num_tiles * p.splits;
    // fewer than 128 rows: load only the rows that exist (the MMA still spans 128 lanes; the
    // lanes beyond M multiply whatever the stage held before and are never read back)
    const int a_rows = a.m >= BM ? BM : ((a.m + 15) / 16) * 16;
    p.a_stage_bytes = a_rows * BK;
    // Two K slabs per stage for the narrowest tiles of an unsplit launch with an even number of slabs: the
    // operands are then described slab by slab ({128 bytes, rows, K/128}) and one copy takes a box two slabs deep.
    const bool two_slabs = BN == 64 && SPLITK == 0 && OUT != kOutQkvHeads && p.splits <= 1 && a.k % (2 * BK) == 0 &&
                           !g_one_slab_stages;
    p.slabs_per_stage = two_slabs ? 2 : 1;

    CUtensorMap tm_a, tm_b;
    if (two_slabs) {
        if (make_map(&tm_a, a.x, BK, (uint64_t)a.m, (uint64_t)(a.k / BK), (uint64_t)a.k, BK, (uint32_t)a_rows, 2)) return 1;
        p.a_kx = 0;
        p.a_kz = 1;
    } else {
        if (make_map(&tm_a, a.x, (uint64_t)a.k, (uint64_t)a.m, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.m,
                     (uint32_t)a_rows))
            return 1;
        p.a_kx = BK;
        p.a_kz = 0;
    }
    if (a.w_layout == B200_W_SLAB128) {
        if (make_map(&tm_b, a.w, BK, (uint64_t)a.n, (uint64_t)(a.k / BK), BK, (uint64_t)a.n * BK, BN, two_slabs ? 2 : 1))
            return 1;
        p.b_kx = 0;
        p.b_kz = 1;
    } else if (two_slabs) {
        if (make_map(&tm_b, a.w, BK, (uint64_t)a.n, (uint64_t)(a.k / BK), (uint64_t)a.k, BK, BN, 2)) return 1;
        p.b_kx = 0;
        p.b_kz = 1;
    } else {
        if (make_map(&tm_b, a.w, (uint64_t)a.k, (uint64_t)a.n, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.n, BN))
            return 1;
        p.b_kx = BK;
        p.b_kz = 0;
    }
    CUtensorMap tm_out;
    memset(&tm_out, 0, sizeof(tm_out));
    if (p.tma_store && make_out_map(&tm_out, a.out, a.out_dtype, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldo))
        return 1;
    cudaError_t le;
    if (SPLITK == 2) {
        // one work item per CTA, `splits` consecutive CTAs form a cluster
        le = launch_kernel_cluster(gemm_i8_kernel<BN, OUT, GENERAL, SPLITK>, dim3(p.num_work), dim3(kThreads),
                                   (size_t)C::kSmemBytes, stream, (unsigned)p.splits, tm_a, tm_b, tm_out, p);
    } else {
        const int grid = p.num_work < di.sms ? p.num_work : di.sms;
        le = launch_kernel(gemm_i8_kernel<BN, OUT, GENERAL, SPLITK>, dim3(grid), dim3(kThreads),
                           (size_t)C::kSmemBytes, stream, tm_a, tm_b, tm_out, p);
    }
    if (le != cudaSuccess) return fail("launching gemm_i8_tcgen05: %s", cudaGetErrorString(le));
    return check_launch("gemm_i8_tcgen05");
}

std::atomic<int> g_pair_mode{0};  // 0 = planner decides, 1 = whenever legal, 2 = never

// Launches the CTA-pair kernel: 256 x 256 tiles, lean epilogue only.
template <int OUT>
int launch_pair(const LinearArgs &a, GemmParams &p, cudaStream_t stream) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    DeviceInfo &di = device_info(dev);
    if (ensure_smem_attr(di.pair_attr_set[OUT], gemm_i8_pair_kernel<OUT>, kPairSmemBytes, "gemm_i8_pair_kernel")) return 1;
    p.num_m_blocks = (a.m + 2 * BM - 1) / (2 * BM);  // 256-row pair blocks
    p.num_n_blocks = (a.n + 255) / 256;
    p.num_tiles = p.num_m_blocks * p.num_n_blocks;
    p.num_k_blocks = (a.k + BK - 1) / BK;
    p.group_m = 16;
    p.splits = 1;
    p.kb_per_split = p.num_k_blocks;
    p.num_work = p.num_tiles;
    p.a_stage_bytes = BM * BK;
    // two K slabs per stage (operands described slab by slab, one copy takes a box two slabs deep) whenever the
    // slab count is even
    const bool two_slabs = a.k % (2 * BK) == 0 && !g_one_slab_stages;
    p.slabs_per_stage = two_slabs ? 2 : 1;
    CUtensorMap tm_a, tm_b, tm_out;
    if (two_slabs) {
        if (make_map(&tm_a, a.x, BK, (uint64_t)a.m, (uint64_t)(a.k / BK), (uint64_t)a.k, BK, BM, 2)) return 1;
        p.a_kx = 0;
        p.a_kz = 1;
    } else {
        if (make_map(&tm_a, a.x, (uint64_t)a.k, (uint64_t)a.m, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.m, BM)) return 1;
        p.a_kx = BK;
        p.a_kz = 0;
    }
    if (a.w_layout == B200_W_SLAB128) {
        if (make_map(&tm_b, a.w, BK, (uint64_t)a.n, (uint64_t)(a.k / BK), BK, (uint64_t)a.n * BK, 128, two_slabs ? 2 : 1))
            return 1;
        p.b_kx = 0;
        p.b_kz = 1;
    } else if (two_slabs) {
        if (make_map(&tm_b, a.w, BK, (uint64_t)a.n, (uint64_t)(a.k / BK), (uint64_t)a.k, BK, 128, 2)) return 1;
        p.b_kx = 0;
        p.b_kz = 1;
    } else {
        if (make_map(&tm_b, a.w, (uint64_t)a.k, (uint64_t)a.n, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.n, 128))
            return 1;
        p.b_kx = BK;
        p.b_kz = 0;
    }
    if (make_out_map(&tm_out, a.out, a.out_dtype, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldo)) return 1;
    const int max_pairs = di.sms / 2;
    const int pairs = p.num_tiles < max_pairs ? p.num_tiles : max_pairs;
    cudaError_t le = launch_kernel_cluster(gemm_i8_pair_kernel<OUT>, dim3(2 * pairs), dim3(kThreads),
                                           (size_t)kPairSmemBytes, stream, 2u, tm_a, tm_b, tm_out, p);
    if (le != cudaSuccess) return fail("launching gemm_i8_pair: %s", cudaGetErrorString(le));
    return check_launch("gemm_i8_pair");
}

template <int BN, int OUT>
int launch_bn(const LinearArgs &a, GemmParams &p, int slot, cudaStream_t stream) {
    if (p.splits > 1 && p.split_mode == 2) return launch_bn_g<BN, OUT, true, 2>(a, p, slot, stream);
    if (p.splits > 1) return launch_bn_g<BN, OUT, true, 1>(a, p, slot, stream);
    const bool lean = p.tma_store && p.vec_ok && (a.n % 32 == 0);
    return lean ? launch_bn_g<BN, OUT, false, 0>(a, p, slot, stream)
                : launch_bn_g<BN, OUT, true, 0>(a, p, slot, stream);
}

// Tuning / test overrides of the planner (process-wide, meant to be set from one thread while no
// other thread launches): tile width, K-split count and split form; 0 = the cost model decides.
std::atomic<int> g_force_bn{0}, g_force_splits{0}, g_force_mode{0};
std::atomic<unsigned long long *> g_trace{nullptr};  // device buffer for per-CTA timestamps (B200_TRACE builds)

}  // namespace

void gemm_set_tile_width(int bn) { gemm_force_plan(bn, 0, 0); }
void gemm_force_plan(int bn, int splits, int mode) {
    g_force_bn = bn;
    g_force_splits = splits;
    g_force_mode = mode;
}
int gemm_forced_tile_width() { return g_force_bn; }
void gemm_set_pair_mode(int mode) { g_pair_mode = mode; }
void gemm_set_one_slab_stages(int on) { g_one_slab_stages = on != 0; }
void gemm_set_trace_buffer(unsigned long long *dev_buf) { g_trace = dev_buf; }
unsigned long long *gemm_trace_buffer() { return g_trace; }

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

namespace {

constexpr size_t kCounterBytes = 4096;  // ticket counters at the head of the workspace (1024 tiles)

struct Plan {
    int bn = 256;
    int splits = 1;
    int mode = 0;  // 0 no split, 1 workspace split-K, 2 cluster split-K
};

// Picks the tile width and the K split from a small time model (microseconds).  A tile costs
// its K slabs (bounded by the MMA rate and by how fast one SM can pull operands through L2),
// its epilogue and, when K is split, the partial-sum exchange; tiles run in waves over the SMs.
// Splitting K inside a cluster needs no scratch and costs two cluster barriers; splitting
// through the global workspace costs fences and a serial read-back and only pays for very long K.
Plan make_plan(int m, int k, int n, int sms, bool allow_workspace) {
    const int mb = (m + BM - 1) / BM;
    const int kblocks = (k + BK - 1) / BK;
    const double a_kb = (m >= BM ? BM : ((m + 15) / 16) * 16) * (double)BK / 1024.0;
    Plan best;
    double best_t = 1e30;
    const int widths[3] = {256, 128, 64};
    for (int wi = 0; wi < 3; ++wi) {
        const int bn = widths[wi];
        const long long tiles = (long long)mb * ((n + bn - 1) / bn);
        for (int mode = 0; mode <= 2; ++mode) {
            if (mode == 1 && !(allow_workspace && (n % 4) == 0 && tiles <= 1024)) continue;
            const int max_splits = mode == 0 ? 1 : 8;
            for (int sp = (mode == 0 ? 1 : 2); sp <= max_splits; ++sp) {
                if (sp > 1 && kblocks / sp < 2) break;
                // a cluster split hands each CTA a whole number of 32-column chunks and of K slabs
                if (mode == 2 && (bn % (32 * sp) != 0 || kblocks % sp != 0)) continue;
                const long long work = tiles * sp;
                if (sp > 1 && work > sms) break;  // keep all partials of a launch in one wave
                const int kbps = (kblocks + sp - 1) / sp;
                const double waves = (double)((work + sms - 1) / sms);
                const double t_mma = 0.065 * bn / 64.0;
                // one SM pulls ~150 KB/us through L2, but with ~100+ CTAs marching over the same
                // A tiles a K slab has not been seen to take less than ~0.3 us (measured)
                double t_load = (a_kb + bn * (double)BK / 1024.0) / 150.0;
                if (t_load < 0.30) t_load = 0.30;
                const double t_epi = 0.45 * bn / 64.0 / (mode == 2 ? sp : 1);
                // cluster exchange: (sp-1)/sp of a 128 x bn int32 tile per CTA at ~20 KB/us (measured)
                const int live_quarters = m >= BM ? 4 : (m + 31) / 32;  // 32-row groups that hold real rows
                const double t_red = mode == 1 ? 3.0 + 1.0 * sp * bn / 64.0
                                               : (mode == 2 ? 1.0 + (sp - 1.0) / sp * bn * 0.0256 * live_quarters / 4.0 : 0.0);
                const double t = waves * (0.3 + kbps * (t_mma > t_load ? t_mma : t_load) + t_epi + t_red);
                if (t < best_t) {
                    best_t = t;
                    best.bn = bn;
                    best.splits = sp;
                    best.mode = mode;
                }
            }
        }
    }
    return best;
}

}  // namespace

size_t gemm_workspace_size(int m, int k, int n) {
    if (m <= 0 || k <= 0 || n <= 0) return 0;
    const Plan pl = make_plan(m, k, n, device_sms(), true);
    return pl.mode == 1 ? kCounterBytes + (size_t)pl.splits * (size_t)m * (size_t)n * sizeof(int32_t) : 0;
}

namespace {
int gemm_launch_impl(const LinearArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream,
                     const Plan *fixed_plan, bool may_allocate);
}

int gemm_launch(const LinearArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream) {
    return gemm_launch_impl(a, workspace, workspace_bytes, stream, nullptr, true);
}

namespace {
void fill_launch_controls(GemmParams &p, bool may_allocate) {
    p.trace = g_trace;
    p.status = status_slot(may_allocate);
    p.wait_limit_ns = wait_limit_ns();
    p.debug_drop_a_load = take_debug_drop();
}

int gemm_launch_impl(const LinearArgs &a, void *workspace, size_t workspace_bytes, cudaStream_t stream,
                     const Plan *fixed_plan, bool may_allocate) {
    if (gemm_can_implement(a, true)) return 1;
    GemmParams p{};
    p.M = a.m; p.N = a.n; p.K = a.k;
    p.row_scales = a.row_scales; p.col_scales = a.col_scales; p.bias = a.bias; p.gate = a.gate;
    p.residual = a.residual; p.ldr = a.ldr; p.out = a.out; p.ldo = a.ldo;
    p.out_dtype = a.out_dtype; p.act = a.out_dtype == B200_DT_S32 ? 0 : a.act;
    fill_launch_controls(p, may_allocate);
    p.static_weights = a.static_weights;
    const size_t esz = (a.out_dtype == B200_DT_S32 || a.out_dtype == B200_DT_F32) ? 4 : 2;
    p.tma_store = aligned16(a.out) && ((a.ldo * esz) % 16 == 0);
    p.vec_ok = (!a.residual || (aligned16(a.residual) && ((a.ldr * esz) % 16 == 0))) &&
               (a.out_dtype == B200_DT_S32 ||
                (aligned16(a.col_scales) && (!a.bias || aligned16(a.bias)) && (!a.gate || aligned16(a.gate))));

    const bool ws_ok = workspace && aligned16(workspace);
    Plan pl = make_plan(a.m, a.k, a.n, device_sms(), ws_ok);
    int force_bn = g_force_bn, force_splits = g_force_splits, force_mode = g_force_mode;
    if (fixed_plan) {
        force_bn = fixed_plan->bn;
        force_splits = fixed_plan->splits;
        force_mode = fixed_plan->mode;
    }
    if (force_bn == 256 || force_bn == 128 || force_bn == 64) pl.bn = force_bn;
    if (force_splits >= 1) {
        pl.splits = force_splits;
        pl.mode = force_splits == 1 ? 0 : (force_mode == 2 ? 2 : 1);
    }
    if (pl.mode == 1) {
        // every K range must hold at least one slab (an empty range would hand the reduction an
        // accumulator that no MMA wrote): at most 8 ranges, and ceil(kblocks / splits) * (splits - 1) < kblocks
        const int kblocks = (a.k + BK - 1) / BK;
        if (pl.splits > 8) pl.splits = 8;
        while (pl.splits > 1 && ((kblocks + pl.splits - 1) / pl.splits) * (pl.splits - 1) >= kblocks) --pl.splits;
        if (pl.splits == 1) pl.mode = 0;
    }
    if (pl.mode == 2) {
        const int kblocks = (a.k + BK - 1) / BK;
        if (pl.bn % (32 * pl.splits) != 0 || kblocks % pl.splits != 0 || pl.splits > 8)
            return fail("cluster split-K needs BN/splits >= 32 and K blocks divisible by splits (bn=%d splits=%d)",
                        pl.bn, pl.splits);
    }
    if (pl.mode == 1) {
        const size_t need = kCounterBytes + (size_t)pl.splits * (size_t)a.m * (size_t)a.n * sizeof(int32_t);
        const long long tiles = (long long)((a.m + BM - 1) / BM) * ((a.n + pl.bn - 1) / pl.bn);
        if (!ws_ok || workspace_bytes < need || tiles > 1024 || (a.n % 4) != 0) {
            if (force_splits > 1) return fail("split-K needs %zu bytes of workspace, got %zu", need, workspace_bytes);
            pl = make_plan(a.m, a.k, a.n, device_sms(), false);
            if (force_bn == 256 || force_bn == 128 || force_bn == 64) pl.bn = force_bn;
        } else {
            p.ws_counters = reinterpret_cast<int *>(workspace);
            p.ws_partials = reinterpret_cast<int32_t *>(reinterpret_cast<char *>(workspace) + kCounterBytes);
        }
    }
    p.splits = pl.splits;
    p.split_mode = pl.mode;
    // CTA pairs: lean epilogue, unsplit 256 x 256 tiles, at least two row blocks.  With two K slabs per stage
    // (K a multiple of 256) the pair kernel measured 7 - 12 % faster than the single-CTA kernel on the wide and
    // the deep linears of an 8192-row band, weights streamed from HBM (QKV 81.8 -> 78.1 us, down 116.4 -> 102.3).
    // With warm weights it already wins from 96 pair tiles of 16 slabs, but with cold weights and few tiles per
    // pair its longer fill (64 KB per CTA before the first MMA, a cluster launch) eats that: M=2048 is neutral in
    // the chained stack and the 2048 x 2048 linears of a band are 3 % behind.  Hence the threshold in pair tiles
    // x K slabs.  With one slab per stage it only pays once the grid runs many waves.
    const bool no_forced_plan = force_bn == 0 && force_splits == 0;
    const bool pair_legal = (pl.bn == 256 || no_forced_plan) && (pl.splits == 1 || no_forced_plan) && a.m > BM &&
                            p.tma_store && p.vec_ok && (a.n % 32 == 0);
    const long long pair_tiles = (long long)((a.m + 255) / 256) * ((a.n + 255) / 256);
    const long long pair_slabs = pair_tiles * ((a.k + BK - 1) / BK);
    const bool pair_two_slabs = a.k % (2 * BK) == 0 && !g_one_slab_stages;
    const bool pair_pays = pair_two_slabs ? pair_slabs >= 2LL * device_sms() * 16 : pair_tiles >= 2 * device_sms();
    const bool pair_wanted = g_pair_mode == 1 || (g_pair_mode == 0 && pair_pays);
    if (pair_legal && pair_wanted && g_pair_mode != 2) {
        p.splits = 1;
        p.split_mode = 0;
        switch (a.out_dtype) {
            case B200_DT_S32: return launch_pair<B200_DT_S32>(a, p, stream);
            case B200_DT_F32: return launch_pair<B200_DT_F32>(a, p, stream);
            case B200_DT_F16: return launch_pair<B200_DT_F16>(a, p, stream);
            default: return launch_pair<B200_DT_BF16>(a, p, stream);
        }
    }
#define B200_LAUNCH(BN_, SLOT_)                                                       \
    switch (a.out_dtype) {                                                            \
        case B200_DT_S32: return launch_bn<BN_, B200_DT_S32>(a, p, SLOT_, stream);    \
        case B200_DT_F32: return launch_bn<BN_, B200_DT_F32>(a, p, SLOT_, stream);    \
        case B200_DT_F16: return launch_bn<BN_, B200_DT_F16>(a, p, SLOT_, stream);    \
        default: return launch_bn<BN_, B200_DT_BF16>(a, p, SLOT_, stream);            \
    }
    if (pl.bn == 256) { B200_LAUNCH(256, 0) }
    if (pl.bn == 128) { B200_LAUNCH(128, 1) }
    B200_LAUNCH(64, 2)
#undef B200_LAUNCH
}
}  // namespace

int linear_qkv_heads(const QkvHeadsArgs &q, cudaStream_t stream) {
    if (q.tokens == 0) return 0;
    if (!q.x || !q.w || !q.row_scales || !q.col_scales || !q.rope_cos || !q.rope_sin || !q.q || !q.k || !q.v ||
        q.tokens < 0 || q.k_dim <= 0 || q.n_heads <= 0 || q.n_kv_heads <= 0)
        return fail("invalid linear_qkv_heads arguments tokens=%d K=%d heads=%d/%d", q.tokens, q.k_dim, q.n_heads,
                    q.n_kv_heads);
    if (q.d_head != kHeadDim)
        return fail("the fused QKV epilogue is built for d_head = %d, got %d (use gemm_i8_i32 + qkv_rms_rope_dequant)",
                    kHeadDim, q.d_head);
    const void *al[] = {q.col_scales, q.rope_cos, q.rope_sin, q.q, q.k, q.v};
    for (const void *ptr : al)
        if (!aligned16(ptr)) return fail("linear_qkv_heads needs 16-byte aligned scales, tables and outputs");
    if (q.bias && !aligned16(q.bias)) return fail("linear_qkv_heads needs a 16-byte aligned bias");
    LinearArgs a{};
    a.x = q.x; a.w = q.w; a.w_layout = q.w_layout; a.m = q.tokens; a.k = q.k_dim;
    a.n = (q.n_heads + 2 * q.n_kv_heads) * kHeadDim;
    a.row_scales = q.row_scales; a.col_scales = q.col_scales; a.bias = q.bias;
    a.out = q.q; a.ldo = a.n; a.out_dtype = B200_DT_F32;  // placeholders for the shared argument check
    a.static_weights = q.static_weights;
    if (gemm_can_implement(a, true)) return 1;
    GemmParams p{};
    p.M = a.m; p.N = a.n; p.K = a.k;
    p.row_scales = a.row_scales; p.col_scales = a.col_scales; p.bias = a.bias;
    p.out_dtype = kOutQkvHeads;
    p.static_weights = a.static_weights;
    fill_launch_controls(p, true);
    p.tma_store = 0;
    p.vec_ok = 1;
    p.splits = 1;
    p.q_heads = q.q; p.k_heads = q.k; p.v_heads = q.v;
    p.rope_cos = q.rope_cos; p.rope_sin = q.rope_sin;
    p.n_heads = q.n_heads; p.n_kv_heads = q.n_kv_heads; p.head_eps = q.eps;
    // 256-wide tiles once they fill the machine, else 128-wide ones for twice the CTAs
    const long long tiles256 = (long long)((a.m + BM - 1) / BM) * ((a.n + 255) / 256);
    int bn = tiles256 >= device_sms() ? 256 : 128;
    const int force_bn = g_force_bn;
    if (force_bn == 256 || force_bn == 128) bn = force_bn;
    if (bn == 256) return launch_bn_g<256, kOutQkvHeads, false, 0>(a, p, 0, stream);
    return launch_bn_g<128, kOutQkvHeads, false, 0>(a, p, 1, stream);
}

int linear_grouped(const GroupedLinear *problems, int count, int w_layout, int act, int out_dtype,
                   cudaStream_t stream, int static_weights) {
    if (count == 0) return 0;
    if (!problems || count < 0) return fail("invalid linear_grouped arguments count=%d", count);
    if (out_dtype != B200_DT_F32 && out_dtype != B200_DT_F16 && out_dtype != B200_DT_BF16)
        return fail("linear_grouped: unsupported output dtype %d", out_dtype);
    if (act < 0 || act > 2) return fail("linear_grouped: unknown activation %d", act);
    if (w_layout != B200_W_SLAB128 && w_layout != B200_W_ROW_MAJOR) return fail("linear_grouped: unknown weight layout");
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    DeviceInfo &di = device_info(dev);
    using C = Cfg<256>;
    const int oi = out_dtype == B200_DT_F32 ? 0 : (out_dtype == B200_DT_F16 ? 1 : 2);
    if (oi == 0 && ensure_smem_attr(di.grouped_attr_set[0], gemm_i8_grouped_kernel<B200_DT_F32>, C::kSmemBytes, "grouped")) return 1;
    if (oi == 1 && ensure_smem_attr(di.grouped_attr_set[1], gemm_i8_grouped_kernel<B200_DT_F16>, C::kSmemBytes, "grouped")) return 1;
    if (oi == 2 && ensure_smem_attr(di.grouped_attr_set[2], gemm_i8_grouped_kernel<B200_DT_BF16>, C::kSmemBytes, "grouped")) return 1;
    const size_t esz = out_dtype == B200_DT_F32 ? 4 : 2;
    static thread_local GroupedParams gp;  // 32 KB: kept off the stack
    static_assert(sizeof(GroupedParams) <= 32764, "kernel parameters are limited to 32 764 bytes");
    // A group larger than one launch can describe is cut into launches of about equal work (tiles x K
    // slabs), not into "as many problems as fit, then the rest": a short last launch leaves most SMs
    // idle for its final round (72 problems of 8 tiles as 48 + 24 ran 5 rounds of tiles for 3.9 rounds of
    // work; as 36 + 36 they run 4).
    const int n_launches = (count + kMaxGroup - 1) / kMaxGroup;
    double total_work = 0.0;
    for (int i = 0; i < count; ++i)
        if (problems[i].n > 0 && problems[i].k > 0)
            total_work += (double)((problems[i].n + 255) / 256) * (double)((problems[i].k + BK - 1) / BK);
    double work_done = 0.0;
    int launch_idx = 0;
    for (int first = 0; first < count; ++launch_idx) {
        int n_here = 0;
        const double target = total_work * (double)(launch_idx + 1) / (double)n_launches;
        const int remaining_launches = n_launches - launch_idx - 1;
        while (first + n_here < count && n_here < kMaxGroup) {
            const GroupedLinear &q = problems[first + n_here];
            const double w = (double)((q.n + 255) / 256) * (double)((q.k + BK - 1) / BK);
            // stop at the work target unless the launches that follow could not hold what would be left
            const bool rest_fits = (long long)(count - first - n_here) <= (long long)remaining_launches * kMaxGroup;
            if (n_here > 0 && work_done + 0.5 * w > target && rest_fits) break;
            work_done += w;
            ++n_here;
        }
        gp.count = n_here; gp.act = act; gp.out_dtype = out_dtype;
        gp.status = status_slot(true);
        gp.wait_limit_ns = wait_limit_ns();
        gp.static_weights = static_weights;
        gp.w_kx = w_layout == B200_W_SLAB128 ? 0 : BK;
        gp.w_kz = w_layout == B200_W_SLAB128 ? 1 : 0;
        int tiles = 0;
        for (int i = 0; i < n_here; ++i) {
            const GroupedLinear &q = problems[first + i];
            if (!q.x || !q.w || !q.row_scales || !q.col_scales || !q.out || q.m <= 0 || q.n <= 0 || q.k <= 0)
                return fail("linear_grouped: invalid problem %d (M=%d K=%d N=%d)", first + i, q.m, q.k, q.n);
            if (q.m > BM) return fail("linear_grouped takes M <= %d rows per problem, problem %d has %d", BM, first + i, q.m);
            if ((q.k & 31) != 0 || (w_layout == B200_W_SLAB128 && (q.k % BK) != 0))
                return fail("linear_grouped: problem %d: K=%d must be a multiple of 32 (128 for the slab layout)", first + i, q.k);
            if (!aligned16(q.x) || !aligned16(q.w)) return fail("linear_grouped: problem %d: x and w must be 16-byte aligned", first + i);
            if (q.ldo < q.n || (q.residual && q.ldr < q.n)) return fail("linear_grouped: problem %d: row stride smaller than N", first + i);
            const int a_rows = ((q.m + 15) / 16) * 16;
            GroupedProblem &d = gp.prob[i];
            d.row_scales = q.row_scales; d.col_scales = q.col_scales; d.bias = q.bias;
            if (q.ldo > 0x7fffffffLL || q.ldr > 0x7fffffffLL || (q.k + BK - 1) / BK > 0xffff)
                return fail("linear_grouped: problem %d: row strides must be below 2^31 elements and K below 8 388 480", first + i);
            d.residual = q.residual; d.out = q.out; d.ldo = (int)q.ldo; d.ldr = (int)q.ldr;
            d.m = q.m; d.n = q.n; d.k_blocks = (unsigned short)((q.k + BK - 1) / BK);
            d.tile0 = tiles;
            d.vec_ok = (!q.residual || (aligned16(q.residual) && ((q.ldr * esz) % 16 == 0))) && aligned16(q.col_scales) &&
                       (!q.bias || aligned16(q.bias));
            tiles += (q.n + 255) / 256;
            d.tma_store = aligned16(q.out) && ((q.ldo * esz) % 16 == 0);
            memset(&gp.tm_out[i], 0, sizeof(CUtensorMap));
            if (d.tma_store && make_out_map(&gp.tm_out[i], q.out, out_dtype, (uint64_t)q.n, (uint64_t)q.m, (uint64_t)q.ldo))
                return 1;
            const uint64_t K = (uint64_t)q.k;
            if (make_map(&gp.tm_a[i], q.x, K, (uint64_t)q.m, 1, K, K * (uint64_t)q.m, (uint32_t)a_rows)) return 1;
            if (w_layout == B200_W_SLAB128) {
                if (make_map(&gp.tm_w[i], q.w, BK, (uint64_t)q.n, (uint64_t)(q.k / BK), BK, (uint64_t)q.n * BK, 256)) return 1;
            } else {
                if (make_map(&gp.tm_w[i], q.w, K, (uint64_t)q.n, 1, K, K * (uint64_t)q.n, 256)) return 1;
            }
        }
        gp.total_tiles = tiles;
        const int grid = tiles < di.sms ? tiles : di.sms;
        cudaError_t le;
        if (oi == 0) le = launch_kernel(gemm_i8_grouped_kernel<B200_DT_F32>, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, stream, gp);
        else if (oi == 1) le = launch_kernel(gemm_i8_grouped_kernel<B200_DT_F16>, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, stream, gp);
        else le = launch_kernel(gemm_i8_grouped_kernel<B200_DT_BF16>, dim3(grid), dim3(kThreads), (size_t)C::kSmemBytes, stream, gp);
        if (le != cudaSuccess) return fail("launching gemm_i8_grouped: %s", cudaGetErrorString(le));
        if (check_launch("gemm_i8_grouped")) return 1;
        first += n_here;
    }
    return 0;
}

size_t static_scratch_capacity() { return kStaticScratchBytes; }

int linear_static_scratch(const LinearArgs &a, cudaStream_t stream) {
    if (gemm_can_implement(a, true)) return 1;
    // The array's name is only a host-side handle; the kernel needs the device address, which is
    // looked up once per device, with that device current.
    static void *scratch_addr[64] = {};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return fail("cudaGetDevice failed");
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!scratch_addr[dev]) {
            void *ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
            if (e != cudaSuccess || !ptr) return fail("cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
            scratch_addr[dev] = ptr;
        }
        scratch = scratch_addr[dev];
    }
    // This entry point always splits K (that is what needs the scratch): the planner's split
    // if it chose one, else two halves.
    const int kblocks = (a.k + BK - 1) / BK;
    if (kblocks < 4 || (a.n % 4) != 0)
        return fail("the no-allocation linear needs K >= 512 and N %% 4 == 0, got K=%d N=%d", a.k, a.n);
    Plan pl = make_plan(a.m, a.k, a.n, device_sms(), true);
    if (pl.mode != 1) {
        pl = Plan();
        pl.bn = a.m <= 128 ? 64 : 128;
        pl.splits = 2;
    }
    pl.mode = 1;  // this entry point is the workspace form of split-K by definition
    const long long tiles = (long long)((a.m + BM - 1) / BM) * ((a.n + pl.bn - 1) / pl.bn);
    auto scratch_needed = [&](int splits) {
        return kCounterBytes + (size_t)splits * (size_t)a.m * (size_t)a.n * sizeof(int32_t);
    };
    while (pl.splits > 2 && scratch_needed(pl.splits) > kStaticScratchBytes) --pl.splits;  // fewer, longer K ranges
    const size_t need = scratch_needed(pl.splits);
    if (need > kStaticScratchBytes || tiles > 1024)
        return fail("M=%d N=%d with %d K-splits needs %zu bytes of scratch; the built-in scratch holds %zu "
                    "(use b200_w8a8_linear with a caller-allocated workspace instead)",
                    a.m, a.n, pl.splits, need, kStaticScratchBytes);
    return gemm_launch_impl(a, scratch, kStaticScratchBytes, stream, &pl, false);
}

// After a launch that gave up a wait, tiles of a split-K launch may have left tickets behind in
// the built-in scratch; a later call would then take an early "last ticket".  Caller-owned
// workspaces are the caller's to zero again.
void gemm_reset_static_tickets() {
    void *ptr = nullptr;
    if (cudaGetSymbolAddress(&ptr, g_static_scratch) == cudaSuccess && ptr) cudaMemset(ptr, 0, kCounterBytes);
    else cudaGetLastError();
}

}  // namespace b200
