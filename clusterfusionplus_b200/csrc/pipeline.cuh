// Thin PTX wrappers for sm_100a: mbarrier, TMA bulk-tensor loads, cache-bypassing
// global loads, and bounded waits.  Every wait in this library goes through
// wait_bounded(): it gives up after a wall-clock limit, raises the CTA's abort
// flag and records a status code, so a stuck barrier ends the kernel with an
// error the host can read instead of hanging the device.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace cfb {

// status codes written to the device status word (0 = OK)
enum : int {
    ST_OK = 0,
    ST_TIMEOUT_FULL = 1,    // consumer never saw a TMA stage land
    ST_TIMEOUT_EMPTY = 2,   // producer never got a stage back
    ST_TIMEOUT_GRID = 3,    // grid-wide barrier did not complete
    ST_TIMEOUT_CLUSTER = 4, // cluster exchange barrier did not complete
    ST_BAD_SEQ = 5,         // seq_len outside [0, kv_rows)
    ST_TIMEOUT_DRAIN = 6,   // copies still in flight at exit after an abort
    ST_TIMEOUT_PEER = 7,    // tensor-parallel peer flag never arrived
};

// Wait limits are staggered so that the wait that names the root cause gives up first: a peer
// GPU that never answers (1.0 s) before the barriers that then cannot complete (1.5 s) before
// the TMA ring, which stalls behind everything else (2.0 s).
constexpr unsigned long long WAIT_LIMIT_NS = 2000ull * 1000ull * 1000ull;
__device__ __forceinline__ unsigned long long wait_limit_ns(int code) {
    return code == 7 ? 1000ull * 1000ull * 1000ull : (code == 3 || code == 4) ? 1500ull * 1000ull * 1000ull : WAIT_LIMIT_NS;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_inval(uint32_t bar) {
    asm volatile("mbarrier.inval.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// acquire at cluster scope: pairs with a peer CTA's release-arrive
__device__ __forceinline__ bool mbar_try_wait_cluster(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Shared abort state of one CTA.
struct AbortCtl {
    volatile int* flag;  // in shared memory
    int* status;         // in global memory
};

__device__ __forceinline__ void raise_abort(const AbortCtl& a, int code) {
    *a.flag = 1;
    atomicCAS(a.status, 0, code);
}

// Pause between two probes of a word in global memory that has not arrived yet, in nanoseconds
// (CFB200_POLL_BACKOFF_NS overrides it when the library first touches a device).
__constant__ int c_poll_backoff_ns = 96;

// Spin on `probe()` until it returns true, the CTA has aborted, or the time
// limit passes.  Returns false when the wait was abandoned.
// BACKOFF_NS > 0 sleeps between probes: for polls of global memory, where many waiting threads
// would otherwise load the L2 (and the data arriving over NVLink) with re-reads.
template <int BACKOFF_NS = 0, class Probe>
__device__ __forceinline__ bool wait_bounded(Probe probe, const AbortCtl& a, int code) {
    if (probe()) return true;
    if (*a.flag) return false;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t it = 0;
    constexpr uint32_t CHECK_MASK = BACKOFF_NS > 0 ? 0xfu : 0xffu;
    while (!probe()) {
        if constexpr (BACKOFF_NS > 0) __nanosleep(c_poll_backoff_ns);
        if ((++it & CHECK_MASK) == 0) {
            if (*a.flag) return false;
            if (globaltimer_ns() - t0 > wait_limit_ns(code)) {
                raise_abort(a, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const AbortCtl& a, int code) {
    return wait_bounded([&] { return mbar_try_wait(bar, parity); }, a, code);
}

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}

// 2-D tiled bulk-tensor load global -> this CTA's shared memory; completion is
// signalled as transaction bytes on `bar`.  x is the innermost coordinate and
// x * element size must be a multiple of 16 bytes.  No multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%2, %3}], [%4], %5;"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar), "l"(policy)
        : "memory");
}

__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---------------------------------------------------------------- global memory
// Loads that skip L1: used for everything another CTA wrote during this kernel.
__device__ __forceinline__ float ld_cg_f32(const float* p) { return __ldcg(p); }
__device__ __forceinline__ float2 ld_cg_f32x2(const float* p) { return __ldcg(reinterpret_cast<const float2*>(p)); }
__device__ __forceinline__ float4 ld_cg_f32x4(const float* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ uint4 ld_cg_u32x4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ __half ld_cg_f16(const __half* p) {
    unsigned short u = __ldcg(reinterpret_cast<const unsigned short*>(p));
    return __ushort_as_half(u);
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// named barrier over the helper warps only
__device__ __forceinline__ void helper_sync(int nthreads) {
    asm volatile("bar.sync 2, %0;" ::"r"(nthreads) : "memory");
}

// named barrier over the helper warps that finish attention partials
__device__ __forceinline__ void fin_sync() {
    asm volatile("bar.sync 3, 64;" ::: "memory");
}

// named barrier over the consumer warps only (the producer warp never joins)
__device__ __forceinline__ void consumer_sync(int nthreads) {
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

}  // namespace cfb
