// 128 x 128 blockwise W8A8: the accuracy option the reference's notes name as their next step
// (docs/cuda_w8a8_optimization.md:319-321 for the rule, :355-356 for the plan).  Activations and
// weights both carry one scale per 128 x 128 block,
//     scale = max(amax, 1e-8) / 128,   code = rne(x / scale) saturated to [-128, 127],
// and the GEMM turns the int32 partial sum of every K block into fp32 with that K block's pair of
// scales before adding it to an fp32 accumulator:
//     y = 0;  for kb in order:  y = fma(float(acc_kb[m, n]), sa[m / 128, kb] * sw[n / 128, kb], y)
// (the scale pair's product rounded to fp32 first, then one fused multiply-add per K block, in fp32),
// then the row/channel linear's epilogue (+ bias, activation, * gate, + residual) and one rounding to the
// output type -- the reference's notes ask for exactly that: block scales inside the fused WorldDiT epilogues.
// The reference tree holds no implementation of this rule (its authors ported a third-party kernel
// out of tree), so parity here is against this library's own CPU restatement of the rule only.
//
// Kernel shape: a 128 x 128 or 128 x 256 output tile per persistent CTA, so a warp's columns see exactly one
// activation block row and one weight block row and a K block's scale pair is a single number per warp (per
// thread when the activations carry a scale per token row, the 1 x 128 form).  The
// tensor core writes K block after K block into the accumulators of tensor memory in turn (four of 128 columns
// or two of 256); eight epilogue warps drain each one as soon as it is complete (`tcgen05.ld` in chunks of 16
// columns, the next chunk in flight while the current one is folded in; the slot is handed back when the last
// chunk has landed) and accumulate in fp32 registers with two-wide instructions, while the next K blocks are
// already running.  int32 -> fp32 is one integer add and one float subtract (|acc| <= 2^21 fits the mantissa of
// 1.5 * 2^23), which keeps the conversion off the 16-lane conversion unit.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "gemm_i8_common.cuh"

namespace b200 {
namespace {

constexpr int BQ = 128;                   // block edge
constexpr int kBqEpilogueWarps = 8;       // two per tensor-memory sub-partition, half of the tile's columns each
constexpr int kBqThreads = 64 + 32 * kBqEpilogueWarps;
constexpr int kBqStagePerWarp = 2048;     // one 32-row x 64-byte block of output per warp
constexpr int kBqStagingBytes = kBqEpilogueWarps * kBqStagePerWarp;

// BN = 128: one weight block per tile (more tiles: small problems); BN = 256: two weight blocks per tile, the
// operand pipeline of the row/channel kernel's widest tile (half the A traffic and half the copies per unit of
// work), chosen whenever it still fills the machine.
template <int BN>
struct BqCfg {
    static constexpr int kStageBytes = BM * BK + BN * BK;
    static constexpr int kStages = BN == 256 ? 4 : 6;
    static constexpr int kSlots = 512 / BN;                      // K-block accumulators: all 512 columns
    static constexpr int kColsPerWarp = BN / 2;                  // 64 or 128: within one weight block
    static constexpr int kChunks = kColsPerWarp / 32;            // output blocks of 32 columns per warp
    static constexpr int kBarBytes = (2 * kStages + kSlots) * 8 + 16;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBqStagingBytes + kBarBytes + 1024;
};
static_assert(BqCfg<128>::kSmemBytes <= 227 * 1024 && BqCfg<256>::kSmemBytes <= 227 * 1024, "shared memory");

// Two fp32 values in one 64-bit register and the two-wide fused multiply-add on them: half the instructions of
// the scalar form, each half rounded like the scalar instruction.  (A two-wide multiply followed by a two-wide
// add is not an alternative where separate roundings are wanted: the assembler merges the pair into the fused
// form even when both carry an explicit rounding mode.)
__device__ __forceinline__ uint64_t pack2(uint32_t lo, uint32_t hi) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, uint32_t &lo, uint32_t &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=r"(lo), "=r"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t add2_rn(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t fma2_rn(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}

// 32 lanes x 16 consecutive 32-bit columns of tensor memory: thread t of the warp receives lane (base + t).
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

struct BlocksParams {
    GemmParams g;            // shape, raster, output, epilogue inputs, wait controls
    const float *a_scales;   // [ceil(M / 128)][K / 128], or [M][K / 128] when every token row has its own
    int a_scale_per_row;     // 1: one activation scale per row and K block (1 x 128 groups)
    const float *w_scales;   // [ceil(N / 128)][K / 128]
    int w_scale_rows;        // ceil(N / 128)
};

// One 32-row x 32-column block of the output: every thread writes its row into the warp's swizzled 2 KB staging
// block, lane 0 hands it to the TMA store engine (which clips at the M / N edges).  A 32-bit block goes as two
// halves of 16 columns through the same staging block.  Once per tile, so the stores are not overlapped.
template <int OUT>
__device__ __forceinline__ void store_block32(const CUtensorMap *tm_out, uint8_t *buf, const uint32_t (&w)[32], int lane,
                                              int row0, int col0) {
    constexpr bool k32 = OUT == B200_DT_F32;
    uint8_t *rowp = buf + lane * 64;
#pragma unroll
    for (int h = 0; h < (k32 ? 2 : 1); ++h) {
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            uint4 val;
            if (k32) {
                val = make_uint4(w[16 * h + 4 * c], w[16 * h + 4 * c + 1], w[16 * h + 4 * c + 2], w[16 * h + 4 * c + 3]);
            } else {
                constexpr int O = Out16<OUT>::value;
                val = make_uint4(OutElem<O>::pack(__uint_as_float(w[8 * c + 0]), __uint_as_float(w[8 * c + 1])),
                                 OutElem<O>::pack(__uint_as_float(w[8 * c + 2]), __uint_as_float(w[8 * c + 3])),
                                 OutElem<O>::pack(__uint_as_float(w[8 * c + 4]), __uint_as_float(w[8 * c + 5])),
                                 OutElem<O>::pack(__uint_as_float(w[8 * c + 6]), __uint_as_float(w[8 * c + 7])));
            }
            *reinterpret_cast<uint4 *>(rowp + ((c ^ ((lane >> 1) & 3)) << 4)) = val;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];" ::"l"(tm_out),
                         "r"(col0 + (k32 ? 16 * h : 0)), "r"(row0), "r"(smem_u32(buf))
                         : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
    }
}

template <int OUT, int BN>
__global__ void __launch_bounds__(kBqThreads, 1)
    gemm_i8_blocks128_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
                             const __grid_constant__ CUtensorMap tm_out, const BlocksParams bp) {
    using C = BqCfg<BN>;
    const GemmParams &p = bp.g;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *staging = smem + C::kStages * C::kStageBytes;
    uint64_t *bar_full = reinterpret_cast<uint64_t *>(staging + kBqStagingBytes);
    // done[s]: the MMAs that read stage s have completed.  One commit per K block serves two waiters: the
    // producer (the stage may be refilled) and the epilogue warps (the K block's accumulator is complete).
    uint64_t *bar_done = bar_full + C::kStages;
    uint64_t *bar_tempty = bar_done + C::kStages;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar_tempty + C::kSlots);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const WaitCtx wctx{abort_flag, p.status, p.wait_limit_ns};

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    pdl_trigger();
    if (threadIdx.x == 0) {
        for (int s = 0; s < C::kStages; ++s) {
            mbar_init(&bar_full[s], 1);
            mbar_init(&bar_done[s], 1);
        }
        for (int b = 0; b < C::kSlots; ++b) mbar_init(&bar_tempty[b], kBqEpilogueWarps);
        *abort_flag = 0;
        fence_mbar_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        tma_prefetch_desc(&tm_out);
    }
    if (warp == 1) {
        tmem_alloc(tmem_slot, 512);
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
            pdl_wait();  // the codes of A come from the kernel before this one
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                int m_blk, n_blk;
                decode_tile(p, tile, m_blk, n_blk);
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    ok = mbar_wait_bounded(&bar_done[s], ph ^ 1u, wctx, KS_TIMEOUT_SMEM_EMPTY);
                    if (!ok) break;
                    uint8_t *sa = smem + s * C::kStageBytes;
                    mbar_arrive_expect_tx(&bar_full[s], (uint32_t)(p.a_stage_bytes + BN * BK));
                    // test aid: leaving out the very first A tile makes the MMA issuer's wait run out
                    const bool drop = p.debug_drop_a_load && tile == (int)blockIdx.x && kb == 0;
                    if (!drop) tma_load_3d(sa, &tm_a, &bar_full[s], kb * BK, m_blk * BM, 0);
                    tma_load_3d(sa + BM * BK, &tm_b, &bar_full[s], kb * p.b_kx, n_blk * BN, kb * p.b_kz);
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_i8(BM, BN);
            int s = 0;
            uint32_t ph = 0;
            uint32_t g = 0;  // K blocks issued so far by this CTA: slot g % kSlots, use number g / kSlots
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
                for (int kb = 0; kb < p.num_k_blocks; ++kb, ++g) {
                    const uint32_t slot = g & (C::kSlots - 1);
                    const uint32_t use = (g / C::kSlots) & 1u;
                    ok = mbar_wait_bounded(&bar_tempty[slot], use ^ 1u, wctx, KS_TIMEOUT_TMEM_EMPTY);
                    if (!ok) break;
                    ok = mbar_wait_bounded(&bar_full[s], ph, wctx, KS_TIMEOUT_SMEM_FULL);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint32_t sa = smem_u32(smem + s * C::kStageBytes);
                    const uint64_t da = umma_smem_desc_k128(sa);
                    const uint64_t db = umma_smem_desc_k128(sa + (uint32_t)(BM * BK));
                    const uint32_t d_tmem = tmem_base + slot * (uint32_t)BN;
#pragma unroll
                    for (int j = 0; j < BK / 32; ++j)
                        umma_i8(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (uint32_t)(j != 0));
                    umma_commit(&bar_done[s]);  // the stage may be refilled, and this K block's sums are complete
                    if (++s == C::kStages) { s = 0; ph ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else {
        const int ew = warp - 2;
        const int sub = warp & 3;     // TMEM sub-partition this warp may read
        const int part = ew >> 2;     // which kColsPerWarp of the tile's columns
        uint8_t *stage = staging + ew * kBqStagePerWarp;
        pdl_wait();  // the activation block scales come from the kernel before this one
        uint32_t g = 0;
        int s = 0;        // the stage whose `done` barrier announces K block g
        uint32_t ph = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < p.num_tiles; tile += gridDim.x) {
            int m_blk, n_blk;
            decode_tile(p, tile, m_blk, n_blk);
            const int colbase = n_blk * BN + part * C::kColsPerWarp;
            // this warp's columns lie in one weight block; beyond the last block there is nothing to scale or store
            const int w_blk = min(colbase / BQ, bp.w_scale_rows - 1);
            // the activation scale of this thread's row: shared by the 128-row block, or the row's own
            const long long a_idx = bp.a_scale_per_row ? (long long)min(m_blk * BM + sub * 32 + lane, p.M - 1) : m_blk;
            const float *sa_row = bp.a_scales + a_idx * p.num_k_blocks;
            const float *sw_row = bp.w_scales + (long long)w_blk * p.num_k_blocks;
            uint64_t acc[C::kChunks][16];  // fp32 pairs (columns 2j, 2j+1): the arithmetic below is two-wide
#pragma unroll
            for (int c = 0; c < C::kChunks; ++c)
#pragma unroll
                for (int j = 0; j < 16; ++j) acc[c][j] = 0ull;
            float f_next = __fmul_rn(__ldg(sa_row), __ldg(sw_row));
#pragma unroll 1
            for (int kb = 0; kb < p.num_k_blocks; ++kb, ++g) {
                const uint32_t slot = g & (C::kSlots - 1);
                const float f = f_next;
                if (kb + 1 < p.num_k_blocks) f_next = __fmul_rn(__ldg(sa_row + kb + 1), __ldg(sw_row + kb + 1));
                ok = mbar_wait_bounded(&bar_done[s], ph, wctx, KS_TIMEOUT_TMEM_FULL);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) break;
                if (++s == C::kStages) { s = 0; ph ^= 1u; }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + ((uint32_t)(sub * 32) << 16) + slot * (uint32_t)BN +
                                       (uint32_t)(part * C::kColsPerWarp);
                const uint64_t ff = pack2(__float_as_uint(f), __float_as_uint(f));
                // 16 columns per tensor-memory load, two register buffers: the load of chunk c+1 is in flight while
                // chunk c is folded in; the slot goes back to the tensor core as soon as the last load has landed
                constexpr int kLoads = C::kColsPerWarp / 16;
                uint32_t ra[16], rb[16];
                tmem_ld_32x16(taddr, ra);
#pragma unroll
                for (int c = 0; c < kLoads; ++c) {
                    tmem_ld_wait();
                    if (c + 1 < kLoads) {
                        tmem_ld_32x16(taddr + (uint32_t)(16 * (c + 1)), (c & 1) ? ra : rb);
                    } else {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bar_tempty[slot]);
                    }
                    const uint32_t(&r0)[16] = (c & 1) ? rb : ra;
                    // float(acc) exactly: 1.5 * 2^23 + acc is representable for |acc| <= 2^22 (here <= 2^21)
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        uint64_t &dst = acc[c / 2][(c & 1) * 8 + j];
                        const uint64_t v = add2_rn(pack2(r0[2 * j] + 0x4B400000u, r0[2 * j + 1] + 0x4B400000u),
                                                   pack2(__float_as_uint(-12582912.0f), __float_as_uint(-12582912.0f)));
                        dst = fma2_rn(v, ff, dst);
                    }
                }
            }
            if (!ok) break;
            const int row0 = m_blk * BM + sub * 32;
#pragma unroll
            for (int c = 0; c < C::kChunks; ++c) {
                const int col0 = colbase + 32 * c;
                if (col0 >= p.N) break;  // warp-uniform
                uint32_t w[32];
#pragma unroll
                for (int j = 0; j < 16; ++j) unpack2(acc[c][j], w[2 * j], w[2 * j + 1]);
                // + bias -> activation -> * gate -> + residual, the order and the separate roundings of the
                // row/channel linear's epilogue; once per tile, so plain guarded accesses are cheap enough
                if (p.bias || p.act != B200_ACT_NONE || p.gate || p.residual) {
                    const int row = row0 + lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int col = col0 + j;
                        if (col >= p.N) continue;
                        float t = __uint_as_float(w[j]);
                        if (p.bias) t = __fadd_rn(t, __ldg(p.bias + col));
                        t = apply_act_rt(t, p.act);
                        if (p.gate) t = __fmul_rn(t, __ldg(p.gate + col));
                        if (p.residual && row < p.M) {
                            const long long ri = (long long)row * p.ldr + col;
                            if (OUT == B200_DT_F32) t = __fadd_rn(reinterpret_cast<const float *>(p.residual)[ri], t);
                            else t = __fadd_rn(OutElem<Out16<OUT>::value>::load1(p.residual, ri), t);
                        }
                        w[j] = __float_as_uint(t);
                    }
                }
                store_block32<OUT>(&tm_out, stage, w, lane, row0, col0);
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
        __syncwarp();
    }

    __syncthreads();
    if (*abort_flag) {
        // a wait ran out somewhere: give copies and MMAs already in flight time to land before the shared and
        // tensor memory they target is released
        const unsigned long long t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) {
        }
        __syncthreads();
    }
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---------------------------------------------------------------- the block quantizer
struct BlockScale {
    float scale, inv;
};
__device__ __forceinline__ int block_code(float v, const BlockScale &bs) {
    // correctly rounded v / scale (one reciprocal per block, Markstein's correction step per element),
    // rounded to the nearest-even integer by adding 1.5 * 2^23
    float q;
    if (bs.inv != 0.0f) {
        const float q0 = __fmul_rn(v, bs.inv);
        const float rem = __fmaf_rn(-q0, bs.scale, v);
        q = __fmaf_rn(rem, bs.inv, q0);
    } else {
        q = __fdiv_rn(v, bs.scale);
    }
    const int c = __float_as_int(__fadd_rn(q, 12582912.0f)) - 0x4B400000;
    return max(-128, min(127, c));
}

template <typename T>
struct Load32;
template <>
struct Load32<float> {
    static __device__ __forceinline__ void load(const float *src, float (&v)[32]) {
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float4 t = __ldg(s4 + i);
            v[4 * i] = t.x; v[4 * i + 1] = t.y; v[4 * i + 2] = t.z; v[4 * i + 3] = t.w;
        }
    }
};
template <>
struct Load32<__half> {
    static __device__ __forceinline__ void load(const __half *src, float (&v)[32]) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 t = __ldg(s4 + i);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
                v[8 * i + 2 * k] = f.x;
                v[8 * i + 2 * k + 1] = f.y;
            }
        }
    }
};
template <>
struct Load32<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16 *src, float (&v)[32]) {
        const uint4 *s4 = reinterpret_cast<const uint4 *>(src);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint4 t = __ldg(s4 + i);
            const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // a bf16 is the upper half of an fp32
                v[8 * i + 2 * k] = __uint_as_float(w[k] << 16);
                v[8 * i + 2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
            }
        }
    }
};

// One CTA of 512 threads per 128 x 128 block: four threads per row, 32 contiguous elements each, held in
// registers between the block maximum and the codes, so the input is read once; two CTAs fit an SM.
// PER_ROW: the same rule on 1 x 128 groups (every token row its own scale per K block, scales[rows][K / 128]): the four
// threads of a row share their maximum with two shuffles and the block-wide reduction falls away.
template <typename T, bool PER_ROW>
__global__ void __launch_bounds__(512, 2) quant_blocks128_kernel(const T *__restrict__ x, long long ldx,
                                                                  int8_t *__restrict__ q, long long ldq,
                                                                  float *__restrict__ scales, int rows, int k_blocks) {
    __shared__ float red[16];
    pdl_trigger();
    const int kb = blockIdx.x, mb = blockIdx.y;
    const int r = mb * BQ + (threadIdx.x >> 2);
    const int c0 = kb * BQ + (threadIdx.x & 3) * 32;
    const bool live = r < rows;
    float v[32];
    pdl_wait();
    if (live) {
        Load32<T>::load(x + (long long)r * ldx + c0, v);
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = 0.0f;
    }
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 32; ++j) amax = fmaxf(amax, fabsf(v[j]));
    if (PER_ROW) {
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    } else {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = amax;
        __syncthreads();
        amax = red[0];
#pragma unroll
        for (int i = 1; i < 16; ++i) amax = fmaxf(amax, red[i]);
    }
    BlockScale bs;
    bs.scale = __fmul_rn(fmaxf(amax, 1e-8f), 0.0078125f);  // / 128: exact, the result is a normal number
    bs.inv = bs.scale < 1e30f ? __frcp_rn(bs.scale) : 0.0f;
    if (PER_ROW) {
        if (live && (threadIdx.x & 3) == 0) scales[(long long)r * k_blocks + kb] = bs.scale;
    } else if (threadIdx.x == 0) {
        scales[(long long)mb * k_blocks + kb] = bs.scale;
    }
    if (!live) return;
    uint4 *dst = reinterpret_cast<uint4 *>(q + (long long)r * ldq + c0);
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        uint32_t w[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int b = 16 * i + 4 * k;
            w[k] = (uint32_t)(block_code(v[b], bs) & 0xFF) | ((uint32_t)(block_code(v[b + 1], bs) & 0xFF) << 8) |
                   ((uint32_t)(block_code(v[b + 2], bs) & 0xFF) << 16) |
                   ((uint32_t)(block_code(v[b + 3], bs) & 0xFF) << 24);
        }
        dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// ---------------------------------------------------------------- fused (Ada)RMSNorm -> 1 x 128 group codes
// The Norm -> A8 fusion of the row/channel path (src/world_cuda_ops.cu:129-182 is what that one replaces) with
// the blockwise rule on 1 x 128 groups: one CTA per row, thread t owns the 8-element vectors t, t + 256, ...
// of the row (read once, kept in registers), the sum of squares is accumulated in fp64 and reduced over the CTA,
// the 16 threads that own one 128-column group share its maximum with four shuffles.
template <typename T>
__device__ __forceinline__ void load8(const T *p, float (&v)[8]);
template <>
__device__ __forceinline__ void load8<float>(const float *p, float (&v)[8]) {
    const float4 a = __ldg(reinterpret_cast<const float4 *>(p)), b = __ldg(reinterpret_cast<const float4 *>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half *p, float (&v)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
        v[2 * k] = f.x;
        v[2 * k + 1] = f.y;
    }
}
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16 *p, float (&v)[8]) {
    const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        v[2 * k] = __uint_as_float(w[k] << 16);
        v[2 * k + 1] = __uint_as_float(w[k] & 0xFFFF0000u);
    }
}

struct RmsGroupArgs {
    const void *x;
    long long ldx;
    const float *vec_scale;  // gamma or modulation [cols], nullable
    int scale_is_mod;        // 1: multiply by (1 + vec_scale)
    const float *vec_bias;   // [cols], nullable
    int8_t *q;
    long long ldq;
    float *scales;           // [rows][cols / 128]
    int rows, cols;
    float eps;
    double inv_cols;         // 1 / cols when that is exact (cols a power of two), else 0: divide
};

template <typename T, int NV>
__global__ void __launch_bounds__(256) rms_quant_row_groups_kernel(const RmsGroupArgs a) {
    __shared__ double red[8];
    pdl_trigger();
    const int row = blockIdx.x, t = threadIdx.x;
    const int nvec = a.cols >> 3;
    const T *xrow = reinterpret_cast<const T *>(a.x) + (long long)row * a.ldx;
    float v[NV][8];
    pdl_wait();
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int vi = t + 256 * j;
        if (vi < nvec) {
            load8<T>(xrow + 8 * vi, v[j]);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) v[j][i] = 0.0f;
        }
    }
    double ss = 0.0;
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const double d = (double)v[j][i];
            ss = fma(d, d, ss);
        }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if ((t & 31) == 0) red[t >> 5] = ss;
    __syncthreads();
    double tot = red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) tot += red[i];
    const double mean = a.inv_cols != 0.0 ? tot * a.inv_cols : tot / (double)a.cols;
    const float inv_rms = (float)rsqrt(mean + (double)a.eps);
    const int k_blocks = a.cols >> 7;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int vi = t + 256 * j;
        const bool has = vi < nvec;  // uniform over the 16 threads of a group: groups are whole
        float amax = 0.0f;
        if (has) {
            const int col = 8 * vi;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float u = __fmul_rn(v[j][i], inv_rms);
                if (a.vec_scale) {
                    const float s = __ldg(a.vec_scale + col + i);
                    u = __fmul_rn(u, a.scale_is_mod ? __fadd_rn(1.0f, s) : s);
                }
                if (a.vec_bias) u = __fadd_rn(u, __ldg(a.vec_bias + col + i));
                v[j][i] = u;
                amax = fmaxf(amax, fabsf(u));
            }
        }
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        if (!has) continue;
        BlockScale bs;
        bs.scale = __fmul_rn(fmaxf(amax, 1e-8f), 0.0078125f);
        bs.inv = bs.scale < 1e30f ? __frcp_rn(bs.scale) : 0.0f;
        if ((t & 15) == 0) a.scales[(long long)row * k_blocks + (vi >> 4)] = bs.scale;
        uint32_t w[2];
#pragma unroll
        for (int h = 0; h < 2; ++h)
            w[h] = (uint32_t)(block_code(v[j][4 * h], bs) & 0xFF) | ((uint32_t)(block_code(v[j][4 * h + 1], bs) & 0xFF) << 8) |
                   ((uint32_t)(block_code(v[j][4 * h + 2], bs) & 0xFF) << 16) |
                   ((uint32_t)(block_code(v[j][4 * h + 3], bs) & 0xFF) << 24);
        *reinterpret_cast<uint2 *>(a.q + (long long)row * a.ldq + 8 * vi) = make_uint2(w[0], w[1]);
    }
}

template <typename T>
static cudaError_t launch_rms_groups(const RmsGroupArgs &a, cudaStream_t stream) {
    const int nvec = a.cols / 8;
    const dim3 grid((unsigned)a.rows);
    if (nvec <= 256) return launch_kernel(rms_quant_row_groups_kernel<T, 1>, grid, dim3(256), 0, stream, a);
    if (nvec <= 512) return launch_kernel(rms_quant_row_groups_kernel<T, 2>, grid, dim3(256), 0, stream, a);
    return launch_kernel(rms_quant_row_groups_kernel<T, 4>, grid, dim3(256), 0, stream, a);
}

struct BlocksDeviceInfo {
    bool attr_set[3][2] = {};
};
BlocksDeviceInfo &blocks_device_info(int dev) {
    static BlocksDeviceInfo info[64];
    return info[dev & 63];
}

template <int OUT, int BN>
int launch_blocks128(const Blocks128Args &a, cudaStream_t stream) {
    using C = BqCfg<BN>;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    BlocksDeviceInfo &di = blocks_device_info(dev);
    constexpr int oi = OUT == B200_DT_F32 ? 0 : (OUT == B200_DT_F16 ? 1 : 2);
    if (ensure_smem_attr(di.attr_set[oi][BN == 256], gemm_i8_blocks128_kernel<OUT, BN>, C::kSmemBytes,
                         "gemm_i8_blocks128_kernel"))
        return 1;
    BlocksParams bp;
    memset(&bp, 0, sizeof(bp));
    GemmParams &p = bp.g;
    p.M = a.m;
    p.N = a.n;
    p.K = a.k;
    p.num_m_blocks = (a.m + BM - 1) / BM;
    p.num_n_blocks = (a.n + BN - 1) / BN;
    p.num_tiles = p.num_m_blocks * p.num_n_blocks;
    p.num_k_blocks = a.k / BK;
    p.group_m = 32;
    p.splits = 1;
    p.num_work = p.num_tiles;
    const int a_rows = a.m >= BM ? BM : ((a.m + 15) / 16) * 16;
    p.a_stage_bytes = a_rows * BK;
    p.bias = a.bias;
    p.gate = a.gate;
    p.residual = a.residual;
    p.ldr = a.ldr;
    p.act = a.act;
    p.out = a.out;
    p.ldo = a.ldo;
    p.out_dtype = a.out_dtype;
    p.tma_store = 1;
    p.status = status_slot(true);
    p.wait_limit_ns = wait_limit_ns();
    p.debug_drop_a_load = take_debug_drop();
    bp.a_scales = a.x_scales;
    bp.a_scale_per_row = a.x_scale_per_row ? 1 : 0;
    bp.w_scales = a.w_scales;
    bp.w_scale_rows = (a.n + BQ - 1) / BQ;
    CUtensorMap tm_a, tm_b, tm_out;
    if (make_map(&tm_a, a.x, (uint64_t)a.k, (uint64_t)a.m, 1, (uint64_t)a.k, (uint64_t)a.k * (uint64_t)a.m,
                 (uint32_t)a_rows))
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
    if (make_out_map(&tm_out, a.out, a.out_dtype, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldo)) return 1;
    const int sms = device_sms();
    const int grid = p.num_tiles < sms ? p.num_tiles : sms;
    cudaError_t le = launch_kernel(gemm_i8_blocks128_kernel<OUT, BN>, dim3((unsigned)grid), dim3(kBqThreads),
                                   (size_t)C::kSmemBytes, stream, tm_a, tm_b, tm_out, bp);
    if (le != cudaSuccess) return fail("launching gemm_i8_blocks128: %s", cudaGetErrorString(le));
    return check_launch("gemm_i8_blocks128");
}

// 256-wide tiles whenever they still give every SM a tile (or when forced for a test), else 128-wide ones.
template <int OUT>
int launch_blocks128_any(const Blocks128Args &a, cudaStream_t stream) {
    const int forced = gemm_forced_tile_width();
    const long long wide_tiles = (long long)((a.m + BM - 1) / BM) * ((a.n + 255) / 256);
    const bool wide = forced == 256 || (forced != 128 && forced != 64 && wide_tiles >= device_sms());
    return wide ? launch_blocks128<OUT, 256>(a, stream) : launch_blocks128<OUT, 128>(a, stream);
}

}  // namespace

template <bool PER_ROW>
static cudaError_t launch_quant_blocks(const void *x, int in_dtype, long long ldx, int8_t *q, long long ldq, float *scales,
                                       int rows, int cols, cudaStream_t stream) {
    const dim3 grid((unsigned)(cols / BQ), (unsigned)((rows + BQ - 1) / BQ));
    if (in_dtype == B200_DT_F32)
        return launch_kernel(quant_blocks128_kernel<float, PER_ROW>, grid, dim3(512), 0, stream, (const float *)x, ldx, q,
                             ldq, scales, rows, cols / BQ);
    if (in_dtype == B200_DT_F16)
        return launch_kernel(quant_blocks128_kernel<__half, PER_ROW>, grid, dim3(512), 0, stream, (const __half *)x, ldx,
                             q, ldq, scales, rows, cols / BQ);
    return launch_kernel(quant_blocks128_kernel<__nv_bfloat16, PER_ROW>, grid, dim3(512), 0, stream,
                         (const __nv_bfloat16 *)x, ldx, q, ldq, scales, rows, cols / BQ);
}

int quantize_blocks128(const void *x, int in_dtype, long long ldx, int8_t *q, long long ldq, float *scales, int rows,
                       int cols, int per_row, cudaStream_t stream) {
    if (!x || !q || !scales || rows <= 0 || cols <= 0) return fail("invalid quantize_blocks128 arguments");
    if (cols % BQ != 0) return fail("quantize_blocks128 needs a column count divisible by 128, got %d", cols);
    const size_t esz = in_dtype == B200_DT_F32 ? 4 : 2;
    if (in_dtype != B200_DT_F32 && in_dtype != B200_DT_F16 && in_dtype != B200_DT_BF16)
        return fail("quantize_blocks128 reads fp32, fp16 or bf16");
    if (ldx < cols || ldq < cols || !aligned16(x) || !aligned16(q) || ((size_t)ldx * esz) % 16 != 0 || ldq % 16 != 0)
        return fail("quantize_blocks128 needs 16-byte aligned buffers and row strides (ldx=%lld, ldq=%lld)", ldx, ldq);
    if ((rows + BQ - 1) / BQ > 65535) return fail("quantize_blocks128: more than 65535 block rows");
    const cudaError_t e = per_row ? launch_quant_blocks<true>(x, in_dtype, ldx, q, ldq, scales, rows, cols, stream)
                                  : launch_quant_blocks<false>(x, in_dtype, ldx, q, ldq, scales, rows, cols, stream);
    if (e != cudaSuccess) return fail("launching quant_blocks128: %s", cudaGetErrorString(e));
    return check_launch("quant_blocks128");
}

int rms_norm_quantize_row_blocks128(const void *x, int in_dtype, long long ldx, const float *vec_scale, int scale_is_mod,
                                    const float *vec_bias, int8_t *q, long long ldq, float *scales, int rows, int cols,
                                    float eps, cudaStream_t stream) {
    if (!x || !q || !scales || rows <= 0 || cols <= 0) return fail("invalid rms_norm_quantize_row_blocks128 arguments");
    if (cols % BQ != 0 || cols > 8192)
        return fail("rms_norm_quantize_row_blocks128 needs a column count divisible by 128, at most 8192; got %d", cols);
    if (in_dtype != B200_DT_F32 && in_dtype != B200_DT_F16 && in_dtype != B200_DT_BF16)
        return fail("rms_norm_quantize_row_blocks128 reads fp32, fp16 or bf16");
    const size_t esz = in_dtype == B200_DT_F32 ? 4 : 2;
    if (ldx < cols || ldq < cols || !aligned16(x) || ((size_t)ldx * esz) % 16 != 0 ||
        (reinterpret_cast<uintptr_t>(q) & 7u) != 0 || ldq % 8 != 0)
        return fail("rms_norm_quantize_row_blocks128 needs 16-byte aligned input rows and 8-byte aligned code rows");
    RmsGroupArgs a{};
    a.x = x; a.ldx = ldx; a.vec_scale = vec_scale; a.scale_is_mod = scale_is_mod; a.vec_bias = vec_bias;
    a.q = q; a.ldq = ldq; a.scales = scales; a.rows = rows; a.cols = cols; a.eps = eps;
    a.inv_cols = (cols & (cols - 1)) == 0 ? 1.0 / (double)cols : 0.0;
    cudaError_t e;
    if (in_dtype == B200_DT_F32) e = launch_rms_groups<float>(a, stream);
    else if (in_dtype == B200_DT_F16) e = launch_rms_groups<__half>(a, stream);
    else e = launch_rms_groups<__nv_bfloat16>(a, stream);
    if (e != cudaSuccess) return fail("launching rms_quant_row_groups: %s", cudaGetErrorString(e));
    return check_launch("rms_quant_row_groups");
}

int linear_blocks128(const Blocks128Args &a, cudaStream_t stream) {
    if (!a.x || !a.w || !a.x_scales || !a.w_scales || !a.out) return fail("linear_blocks128: null operand");
    if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail("linear_blocks128: bad shape M=%d K=%d N=%d", a.m, a.k, a.n);
    if (a.k % BK != 0) return fail("linear_blocks128 needs K divisible by 128, got K=%d", a.k);
    if (a.w_layout != B200_W_ROW_MAJOR && a.w_layout != B200_W_SLAB128) return fail("unknown weight layout %d", a.w_layout);
    if (a.out_dtype != B200_DT_F32 && a.out_dtype != B200_DT_F16 && a.out_dtype != B200_DT_BF16)
        return fail("linear_blocks128 writes fp32, fp16 or bf16");
    const size_t esz = a.out_dtype == B200_DT_F32 ? 4 : 2;
    if (!aligned16(a.x) || !aligned16(a.w)) return fail("linear_blocks128: codes must be 16-byte aligned");
    if (a.act != B200_ACT_NONE && a.act != B200_ACT_SILU && a.act != B200_ACT_GELU_TANH) return fail("unknown activation %d", a.act);
    if (a.residual && a.ldr < a.n) return fail("linear_blocks128: residual row stride %lld below N=%d", a.ldr, a.n);
    if (a.ldo < a.n || !aligned16(a.out) || ((size_t)a.ldo * esz) % 16 != 0)
        return fail("linear_blocks128: y must be 16-byte aligned with 16-byte aligned rows (ldo=%lld)", a.ldo);
    switch (a.out_dtype) {
        case B200_DT_F32: return launch_blocks128_any<B200_DT_F32>(a, stream);
        case B200_DT_F16: return launch_blocks128_any<B200_DT_F16>(a, stream);
        default: return launch_blocks128_any<B200_DT_BF16>(a, stream);
    }
}

}  // namespace b200
