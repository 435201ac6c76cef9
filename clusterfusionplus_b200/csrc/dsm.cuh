// Distributed-shared-memory (DSMEM) collectives for one thread-block cluster.
//
// Role: what the reference's include/dsm.cuh:20-171 (`cluster_reduce<>`) does for
// its kernels — summing per-CTA partial vectors across the CTAs of a cluster —
// redesigned:
//   * fp32 end to end (the reference adds fp16 pairs with __hadd2),
//   * a push reduce-scatter instead of a recursive-doubling all-reduce: each
//     CTA stores the slice another CTA owns straight into that CTA's receive
//     buffer (st.shared::cluster), signals it with one release-arrive on an
//     mbarrier in the owner's shared memory, and the owner adds the CS slices
//     in a fixed pairwise tree, so the result does not depend on arrival order,
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

// Reduce-scatter of `nrows` fp32 partials across the CS CTAs of the cluster.
//
//   partial   : this CTA's partial sums, nrows floats, shared memory
//   recv      : this CTA's receive buffer, CS slices of `stride` floats each
//   xbar      : this CTA's exchange mbarrier (initialised with count CS - 1)
//   parity    : phase parity of this use of xbar (caller toggles it per use)
//   tid/nthr  : index of the calling thread among the `nthr` consumer threads
//
// On return recv[c * stride + i] holds CTA c's partial for the row this CTA owns
// at slice index i; the caller sums them with tree_sum<CS>().  All `nthr`
// consumer threads must call it.  Returns false if the wait was abandoned.
template <int CS>
__device__ __forceinline__ bool reduce_scatter_push(const float* partial, float* recv, int stride, int nrows,
                                                    uint64_t* xbar, uint32_t parity, int tid, int nthr,
                                                    const AbortCtl& ab) {
    const uint32_t me = (CS > 1) ? cta_rank() : 0u;
    consumer_sync(nthr);  // partial[] complete
    for (int t = tid; t < nrows; t += nthr) {
        const uint32_t owner = static_cast<uint32_t>(t) % CS;
        float* slot = recv + me * stride + t / CS;
        if (owner == me) {
            *slot = partial[t];
        } else {
            st_remote_f32(map_to_rank(smem_u32(slot), owner), partial[t]);
        }
    }
    if constexpr (CS > 1) {
        consumer_sync(nthr);  // all remote stores of this CTA issued
        if (tid == 0) {
            fence_acq_rel_cluster();
            const uint32_t bar = smem_u32(xbar);
#pragma unroll
            for (uint32_t c = 0; c < CS; ++c)
                if (c != me) arrive_remote_release(map_to_rank(bar, c));
        }
        const uint32_t bar = smem_u32(xbar);
        bool ok = wait_bounded([&] { return mbar_try_wait_cluster(bar, parity); }, ab, ST_TIMEOUT_CLUSTER);
        consumer_sync(nthr);
        return ok;
    } else {
        consumer_sync(nthr);
        return true;
    }
}

}  // namespace dsm
}  // namespace cfb
