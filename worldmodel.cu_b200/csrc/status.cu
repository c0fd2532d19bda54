// The status word that device-side bounded waits report into, and the host side of it.
//
// The reference's operators report every failure as `return 1` plus a message
// (src/world_cuda_ops.cu:28-42, 2856-2863); its kernels cannot fail half-way because they never
// wait on anything.  The tcgen05 kernels here do wait (mbarriers fed by TMA and by other CTAs), with
// a time limit; a wait that runs out leaves a code in a status word and the kernel drains and exits.
// So that the NEXT operator call can return 1 without synchronizing the device, the word lives in
// pinned host memory mapped into the device's address space: the device writes it with a
// system-scope fence, the host reads it with a plain load at the top of every entry point.
#include <mutex>

#include "common.cuh"
#include "w8a8_internal.h"

namespace b200 {

__device__ int g_device_status = 0;  // used while no mapped word exists (callers that may not allocate)

namespace {
std::mutex g_mu;
volatile int *g_mapped_host = nullptr;
int *g_mapped_dev = nullptr;
bool g_map_tried = false;
int *g_symbol_addr[64] = {};
unsigned long long g_wait_limit_ns = kDefaultWaitLimitNs;
int g_drop_a_loads = 0;

const char *status_text(int code) {
    switch (code) {
        case KS_TIMEOUT_SMEM_EMPTY: return "the TMA producer waited too long for a free pipeline stage";
        case KS_TIMEOUT_SMEM_FULL: return "the MMA issuer waited too long for an operand stage";
        case KS_TIMEOUT_TMEM_EMPTY: return "the MMA issuer waited too long for a drained accumulator";
        case KS_TIMEOUT_TMEM_FULL: return "the epilogue waited too long for a finished accumulator";
        case KS_TIMEOUT_ROW_EXCHANGE: return "the epilogue waited too long for the row statistics of its cluster";
        default: return "unknown status";
    }
}
}  // namespace

int *status_slot(bool may_allocate) {
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_mapped_dev && may_allocate && !g_map_tried) {
        g_map_tried = true;
        void *h = nullptr, *d = nullptr;
        // the first launch of a process may sit inside a stream capture, where allocating calls are
        // refused unless the thread's capture mode is relaxed for their duration
        cudaStreamCaptureMode mode = cudaStreamCaptureModeRelaxed;
        cudaThreadExchangeStreamCaptureMode(&mode);
        if (cudaHostAlloc(&h, 64, cudaHostAllocMapped | cudaHostAllocPortable) == cudaSuccess) {
            *reinterpret_cast<volatile int *>(h) = 0;
            if (cudaHostGetDevicePointer(&d, h, 0) == cudaSuccess && d) {
                g_mapped_host = reinterpret_cast<volatile int *>(h);
                g_mapped_dev = reinterpret_cast<int *>(d);
            } else {
                cudaFreeHost(h);
            }
        }
        cudaThreadExchangeStreamCaptureMode(&mode);
        cudaGetLastError();  // a refused mapping is not an error of the caller's launch
    }
    if (g_mapped_dev) return g_mapped_dev;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    if (!g_symbol_addr[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_device_status) == cudaSuccess) g_symbol_addr[dev] = reinterpret_cast<int *>(p);
        else cudaGetLastError();
    }
    return g_symbol_addr[dev];
}

unsigned long long wait_limit_ns() { return g_wait_limit_ns; }
void set_wait_limit_ns(unsigned long long ns) { g_wait_limit_ns = ns ? ns : kDefaultWaitLimitNs; }
void debug_drop_a_loads(int launches) { g_drop_a_loads = launches > 0 ? launches : 0; }
int take_debug_drop() {
    std::lock_guard<std::mutex> lock(g_mu);
    if (g_drop_a_loads <= 0) return 0;
    --g_drop_a_loads;
    return 1;
}

int status_check_entry() {
    volatile int *h = g_mapped_host;
    if (!h || *h == 0) return 0;
    // failure path: let everything queued finish (all waits are bounded), then start clean
    const int code = *h;
    cudaDeviceSynchronize();
    *h = 0;
    gemm_reset_static_tickets();
    return fail("an earlier kernel gave up a bounded wait (status %d: %s); the outputs of that launch are incomplete, "
                "and a split-K workspace it used must be zeroed again before reuse",
                code, status_text(code));
}

int status_poll(int *status_out) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return fail("cudaDeviceSynchronize: %s", cudaGetErrorString(e));
    int st = 0;
    if (g_mapped_host) st = *g_mapped_host;
    int dev_st = 0;
    e = cudaMemcpyFromSymbol(&dev_st, g_device_status, sizeof(int));
    if (e != cudaSuccess) return fail("cudaMemcpyFromSymbol: %s", cudaGetErrorString(e));
    if (st == 0) st = dev_st;
    if (status_out) *status_out = st;
    if (st != 0) {
        if (g_mapped_host) *g_mapped_host = 0;
        const int zero = 0;
        cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int));
        gemm_reset_static_tickets();
    }
    return 0;
}

}  // namespace b200
