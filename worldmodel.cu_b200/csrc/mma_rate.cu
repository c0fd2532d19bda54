// Self-test: how fast this device issues and retires tcgen05.mma kind::i8 when nothing else is in
// the way.  One CTA per SM issues 128 x 256 x 32 MMAs back to back on two resident operand tiles
// (whatever bytes shared memory holds: the integer pipe does not care) with no loads, no barriers
// between them and no epilogue.  The rate is the ceiling any int8 GEMM on this part can approach;
// bench.py reports it as the measured int8 peak next to the nominal figure.  The reference has
// nothing comparable (its GEMM is a CUTLASS mma.sync instantiation, src/world_cuda_ops.cu:529-548).
#include "gemm_i8_common.cuh"

namespace b200 {
namespace {

constexpr int kRateBN = 256;
constexpr int kRateSmem = BM * BK + kRateBN * BK + 1024 + 64;

__global__ void __launch_bounds__(128, 1) mma_issue_rate_kernel(int slabs, int *status, unsigned long long limit_ns) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + BM * BK + kRateBN * BK);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 0) {
        tmem_alloc(tmem_slot, kRateBN);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t d_tmem = *tmem_slot;
    if (warp == 1 && lane == 0) {
        constexpr uint32_t idesc = umma_idesc_i8(BM, kRateBN);
        const uint32_t sa = smem_u32(smem);
        const uint64_t da = umma_smem_desc_k128(sa), db = umma_smem_desc_k128(sa + BM * BK);
        for (int i = 0; i < slabs; ++i) {
#pragma unroll
            for (int j = 0; j < BK / 32; ++j)
                umma_i8(d_tmem, da + (uint64_t)(2 * j), db + (uint64_t)(2 * j), idesc, (uint32_t)((i | j) != 0));
        }
        umma_commit(bar);
        const WaitCtx w{abort_flag, status, limit_ns};
        mbar_wait_bounded(bar, 0, w, KS_TIMEOUT_TMEM_FULL);
    }
    __syncthreads();
    if (warp == 0) {
        tc_fence_after_sync();
        tmem_dealloc(d_tmem, kRateBN);
    }
}

}  // namespace

int mma_issue_rate(int slabs_per_cta, double *tera_ops_per_s) {
    if (slabs_per_cta <= 0 || slabs_per_cta > (1 << 24) || !tera_ops_per_s)
        return fail("mma_issue_rate: slabs_per_cta must be in 1 .. 2^24 and the result pointer non-null");
    static bool attr_set[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return fail("cudaGetDevice failed");
    if (ensure_smem_attr(attr_set[dev & 63], mma_issue_rate_kernel, kRateSmem, "mma_issue_rate_kernel")) return 1;
    const int sms = device_sms();
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (cudaEventCreate(&e0) != cudaSuccess || cudaEventCreate(&e1) != cudaSuccess) return fail("cudaEventCreate failed");
    int *status = status_slot(true);
    const unsigned long long limit = 20000000000ull;  // the whole loop runs under one wait: 20 s
    mma_issue_rate_kernel<<<sms, 128, kRateSmem>>>(slabs_per_cta < 1024 ? slabs_per_cta : 1024, status, limit);  // warm-up
    cudaEventRecord(e0);
    mma_issue_rate_kernel<<<sms, 128, kRateSmem>>>(slabs_per_cta, status, limit);
    cudaEventRecord(e1);
    cudaError_t e = cudaEventSynchronize(e1);
    float ms = 0.0f;
    if (e == cudaSuccess) e = cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    if (e != cudaSuccess || ms <= 0.0f) return fail("mma_issue_rate: %s", cudaGetErrorString(e));
    const double ops = (double)sms * (double)slabs_per_cta * (BK / 32) * 2.0 * BM * kRateBN * 32.0;
    *tera_ops_per_s = ops / ((double)ms * 1e-3) / 1e12;
    return check_launch("mma_issue_rate");
}

}  // namespace b200
