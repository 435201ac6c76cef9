// Distributed-shared-memory (DSMEM) collectives for one thread-block cluster.
//
// Role: what the reference's include/dsm.cuh:20-171 (`cluster_reduce<>`) does for
// its kernels — summing per-CTA partial vectors across the CTAs of a cluster —
// redesigned:
//   * fp32 end to end (the reference adds fp16 pairs with __hadd2),
//   * a push reduce-scatter instead of a recursive-doubling all-reduce: each
//     CTA stores the rows another CTA owns straight into that CTA's receive
//     buffer (st.shared::cluster) from the thread that finished the row, every
//     warp signals with one release-arrive per CTA on an mbarrier in the owner's
//     shared memory, and the owner adds the CS slices in a fixed pairwise tree,
//     so the result does not depend on arrival order,
//   * no hardware cluster barrier on the data path: the only waits are bounded
//     mbarrier waits, so the producer warp that streams weights is never held.
//
// Row t of the cluster's vector is owned by CTA (t % CS) and lives at index
// t / CS of that CTA's slice.
#pragma once
#include "pipeline.cuh"

namespace cfb {
namespace dsm {

__device__ __forceinline__ uint32_t cta_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// address of `local_smem_addr` inside CTA `rank` of this cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_smem_addr), "r"(rank));
    return r;
}

__device__ __forceinline__ void st_remote_f32(uint32_t cluster_addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(cluster_addr), "f"(v) : "memory");
}

__device__ __forceinline__ void arrive_remote_release(uint32_t cluster_bar_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_bar_addr) : "memory");
}

__device__ __forceinline__ void fence_acq_rel_cluster() {
    asm volatile("fence.acq_rel.cluster;" ::: "memory");
}

// Full hardware cluster barrier; every thread of every CTA of the cluster must
// call it.  Used only at kernel start (after mbarrier init) and at kernel end.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// fixed-order tree sum of the CS slices
template <int CS>
__device__ __forceinline__ float tree_sum(const float* recv, int stride, int idx) {
    if constexpr (CS == 1) {
        return recv[idx];
    } else if constexpr (CS == 2) {
        return recv[idx] + recv[stride + idx];
    } else {
        static_assert(CS == 4, "cluster size must be 1, 2 or 4");
        return (recv[idx] + recv[stride + idx]) + (recv[2 * stride + idx] + recv[3 * stride + idx]);
    }
}

// Reduce-scatter of fp32 partial rows across the CS CTAs of the cluster, without a CTA-wide barrier.
//
//   recv      : this CTA's receive buffer, CS slices of `stride` floats each
//   xbar      : this CTA's exchange mbarrier, initialised with count NWARP * CS: every warp of every
//               CTA of the cluster (this one included) arrives once per exchange
//
// The thread that holds the finished partial of row t calls scatter_row(): it stores the value into
// slot [me][t / CS] of the receive buffer of the CTA that owns the row (t % CS) -- its own shared memory
// or, through distributed shared memory, a peer's.  When a warp has scattered all its rows it calls
// exchange_arrive(): one lane release-arrives on every CTA's exchange barrier, which (through the warp
// barrier before it) publishes the warp's stores.  exchange_wait() then returns once all NWARP * CS
// arrivals of this exchange are in: recv[c * stride + i] holds CTA c's partial of the row this CTA owns
// at slice index i, and the caller sums them with tree_sum<CS>().
template <int CS>
__device__ __forceinline__ void scatter_row(float* recv, int stride, uint32_t me, int t, float v) {
    const uint32_t owner = static_cast<uint32_t>(t) % CS;
    float* slot = recv + me * stride + t / CS;
    if (owner == me) {
        *slot = v;
    } else {
        st_remote_f32(map_to_rank(smem_u32(slot), owner), v);
    }
}

template <int CS>
__device__ __forceinline__ void exchange_arrive(uint64_t* xbar, uint32_t me, int lane) {
    __syncwarp();
    if (lane == 0) {
        const uint32_t bar = smem_u32(xbar);
#pragma unroll
        for (uint32_t c = 0; c < CS; ++c) {
            if (c == me) asm volatile("mbarrier.arrive.release.cta.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
            else arrive_remote_release(map_to_rank(bar, c));
        }
    }
}

__device__ __forceinline__ bool exchange_wait(uint64_t* xbar, uint32_t parity, const AbortCtl& ab) {
    const uint32_t bar = smem_u32(xbar);
    return wait_bounded([&] { return mbar_try_wait_cluster(bar, parity); }, ab, ST_TIMEOUT_CLUSTER);
}

}  // namespace dsm
}  // namespace cfb
