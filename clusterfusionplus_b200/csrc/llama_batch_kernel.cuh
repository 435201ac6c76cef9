// Batched Llama decode blocks for sm_100a (up to 16 sequences, one token each): the attention block
// over a paged KV pool and the SwiGLU MLP block, each ONE persistent cooperative launch.
//
// What the reference does in LlamaDecoderLayerBatchDecodeWithPagedKVCacheKernel
// (include/5090/llama/kernel_batch_sglang.cuh:43-664): one 4-CTA cluster per (sequence, head), so
// every weight byte is fetched once per sequence and every partial sum is an fp16 atomicAdd.  Here
// the weights are streamed ONCE per step for all sequences, which turns every projection into a
// skinny GEMM  out[b, n] = sum_k act[b, k] * W[n, k]  with b <= 16, and that runs on the 5th
// generation tensor cores:
//
//   * operands: the weight tile (B operand, N = the CTA's weight rows, K-major, exactly nn.Linear's
//     layout) and the activation tile (A operand, M = 64 rows of which the first `batch` are real) are
//     both brought into shared memory by TMA with the 128-byte swizzle, one copy each per ring stage; one
//     thread issues tcgen05.mma.cta_group::1.kind::f16 (M 64, N = the CTA's rows, K 16 per instruction),
//     alternating between independent accumulator sets so that consecutive K steps do not wait for one
//     another;
//   * accumulators live in tensor memory (fp32, lanes = sequences, columns = weight rows) and are read
//     back once per phase with tcgen05.ld by one warp, which applies the epilogue (store fp32 q/k/v,
//     silu(gate) * up, fp16 output);
//   * tcgen05.commit hands a ring stage back to the TMA producer when the MMAs that read it are done.
//
// The output rows of every projection are split over all CTAs in 8-row granules.  The two narrow projections
// (O and down: under 40 rows per CTA, bound by the NUMBER of MMAs) are in addition cut along K over groups of CTAs:
// fp32 partial outputs in global memory, a grid barrier, the slices added in slice order.  The merged [gate; up]
// matrix is fetched through a 4-D map, so that one copy brings a K block's gate rows followed by its up rows: one
// B operand.  Every sum has a fixed order and nothing is atomic.  Attention streams each sequence's cached rows
// through the page table (the pool row of token t of sequence b is indices[indptr[b] + t], one row =
// one token, as in the reference's `paged_kv_indices[...] * HIDDEN_DIM` addressing, :343-371) with one
// 256-byte run of asynchronous copies per (row, head), in items of 128 rows spread evenly over the CTAs; partial (max,
// denominator, numerators) records are merged in a fixed order, the new token is folded in and
// appended to the pool there.  Phases are separated by grid barriers (bounded waits).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "pipeline.cuh"

namespace cfb {
namespace lb {

constexpr int MAXB = 16;              // sequences per step
constexpr int D = 128;                // head_dim (include/5090/llama/config.h:1)
constexpr int NCW = 8;                // consumer warps (attention arithmetic, norms, merge; warp 0 also the GEMM epilogue)
constexpr int NCT = NCW * 32;
constexpr int NGW = 4;                // warps that gather K/V rows in the attention phase: the TMA warp, the MMA warp, two more
constexpr int THREADS = NCT + NGW * 32;
constexpr int NSTAGE = 4;
constexpr int STAGE_BYTES = 44 * 1024;  // two K blocks of the widest tile (16 + 2 x 80 rows) fit: half the copies per byte
constexpr int A_KB_BYTES = 16 * 128;  // one 64-wide K block of the activation tile: 16 rows x 128 bytes
constexpr int KV_ROWS = 128;          // cache rows per attention item
constexpr int REC = D + 4;            // partial record: D numerators, max, denominator, pad
constexpr int TMEM_COLS = 512;

enum : int { MODE_ATTN = 0, MODE_MLP = 1 };

// One weight matrix [rows, K] as a 3-D tensor {64 K elements, rows, K / 64 blocks}: a box {64, R, kb} brings R
// rows of kb consecutive 64-wide K blocks in ONE copy, landing block-major ([kb][R][128 bytes], 128-byte swizzle),
// which is the K-major operand layout the MMA reads.  The rows of a phase are split over the CTAs in 8-row
// granules, so a CTA holds rows_lo or rows_lo + 8 rows: one map for each.
struct WMaps {
    CUtensorMap lo, hi;
    int rows_lo;  // box rows of `lo`; `hi` has rows_lo + 8
    int kb;       // K blocks per ring stage (box depth of the maps, and of the matching activation map)
    int nset;     // accumulator sets the K steps alternate between (independent MMA chains), summed in the epilogue
    int ksplit;   // > 1: K is cut into ksplit slices over CTAs that share a row group (narrow matrices); partials meet in global memory
};

struct alignas(64) Params {
    WMaps w_qkv, w_o, w_gu, w_down;
    // activations, stored K-block-major [K / 64][16 sequences][64] fp16 so that a stage's tile is one contiguous
    // copy: 2-D maps {64, 16 * K / 64} with box {64, 16 * kb} for the phase that reads them
    CUtensorMap a_qkv, a_o, a_gu, a_down;
    int mode, B, H, NH, F;
    float eps;
    const __half *input, *residual, *norm_w;
    __half *residual_out, *output;
    // attention block
    const int *indptr, *indices;
    const unsigned long long *k_ptrs, *v_ptrs;
    int layer_id;
    const long long* positions;
    const float* cos_sin;  // [positions, 128]: cos of the 64 rotation angles, then sin
    // scratch
    __half *y16, *attn16, *mid16;  // K-block-major activations of H, H and F columns (see a_idx)
    float* qkv32;                  // [16, 3H]
    float* split32;                // [ksplit][16][H] fp32 partial outputs of a K-split projection
    float* records;                // [B * NH + grid][REC]
    unsigned* sync;                // [0] barrier count, [1] exit count
    int* status;
    unsigned long long* trace;     // diagnostics: [grid][16] nanosecond stamps at the phase boundaries, or nullptr
};

// ---------------------------------------------------------------- tcgen05 wrappers
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// D[tmem] (+)= A[smem] * B[smem]^T, fp16 operands, fp32 accumulate; issued by ONE thread
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrive (count 1) on a shared-memory mbarrier once every MMA this thread issued so far has finished
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 8 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor of a K-major operand tile stored with the 128-byte swizzle: rows of
// 128 bytes (64 fp16), groups of 8 rows 1024 bytes apart.  Fields (sm_100): start address >> 4 in bits
// [0,14), leading byte offset >> 4 in [16,30) (1 for swizzled K-major), stride byte offset >> 4 in
// [32,46), descriptor version 1 in [46,48), layout type 2 (128-byte swizzle) in [61,64).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t saddr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((saddr & 0x3ffffu) >> 4);
    d |= static_cast<uint64_t>(1u) << 16;
    d |= static_cast<uint64_t>(1024u >> 4) << 32;
    d |= static_cast<uint64_t>(1u) << 46;
    d |= static_cast<uint64_t>(2u) << 61;
    return d;
}
// Instruction descriptor: fp32 accumulator (bits [4,6) = 1), fp16 A and B (formats 0), both K-major,
// N >> 3 in bits [17,23), M >> 4 in bits [24,29).
__host__ __device__ __forceinline__ uint32_t idesc_f16(int m, int n) {
    return (1u << 4) | (static_cast<uint32_t>(n >> 3) << 17) | (static_cast<uint32_t>(m >> 4) << 24);
}

// element (sequence b, column k) of a K-block-major activation matrix
__host__ __device__ __forceinline__ size_t a_idx(int b, int k) {
    return (static_cast<size_t>(k >> 6) * 16 + b) * 64 + (k & 63);
}

__device__ __forceinline__ void tma3d(uint32_t dst, const void* tmap, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tma4d(uint32_t dst, const void* tmap, int x, int y, int z, int w, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
        : "memory");
}

// 2-D tiled TMA load without cache hint
__device__ __forceinline__ void tma2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar)
        : "memory");
}
// untiled bulk copy global -> shared (size and both addresses multiples of 16 bytes)
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ int pbegin(int i, int total, int parts) {
    return static_cast<int>((static_cast<long long>(i) * total) / parts);
}
__device__ __forceinline__ int pof(int t, int total, int parts) {
    return static_cast<int>(((static_cast<long long>(t) + 1) * parts - 1) / total);
}

__device__ __forceinline__ void csync() { asm volatile("bar.sync 1, %0;" ::"n"(NCT) : "memory"); }

// sum over the consumer threads, broadcast to all of them (red: 16 floats of shared memory)
__device__ __forceinline__ float csum(float v, float* red, int tid) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    csync();
    if ((tid & 31) == 0) red[tid >> 5] = v;
    csync();
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < NCW; ++i) t += red[i];
    return t;
}

struct Ring {
    uint32_t base, full, empty;
    int stage;
    uint32_t phase;
    __device__ __forceinline__ void advance() {
        if (++stage == NSTAGE) {
            stage = 0;
            phase ^= 1u;
        }
    }
};

// ---------------------------------------------------------------- the kernel
__global__ void __launch_bounds__(THREADS, 1) llama_batch_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    // [ring NSTAGE x STAGE_BYTES][q 128 f][merge 16 x 128 f + 32 f][red 32 f][prefix 17 i][barriers][tmem ptr][abort]
    uint8_t* ring = smem_raw;
    float* q_s = reinterpret_cast<float*>(ring + NSTAGE * STAGE_BYTES);
    float* mbuf = q_s + D;             // [16][D]
    float* mlbuf = mbuf + 16 * D;      // [16][2]
    float* red = mlbuf + 32;           // 32
    int* pre = reinterpret_cast<int*>(red + 32);  // [MAXB + 1] item prefix, then [MAXB] seq lens
    uint64_t* bars = reinterpret_cast<uint64_t*>(pre + 2 * MAXB + 2);
    // two sets of ring barriers over the same stages: the GEMM phases release a stage with one
    // tcgen05.commit arrival, the attention phase with one arrival per consumer warp (phases never overlap
    // and each drains its ring, so the stage memory can be shared)
    uint64_t* full = bars;
    uint64_t* empty = bars + NSTAGE;
    uint64_t* full2 = bars + 2 * NSTAGE;
    uint64_t* empty2 = bars + 3 * NSTAGE;
    uint64_t* acc_bar = bars + 4 * NSTAGE;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 4 * NSTAGE + 1);
    int* abort_flag = reinterpret_cast<int*>(tmem_slot + 1);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    const AbortCtl ab{abort_flag, p.status};
    const int B = p.B, H = p.H, NH = p.NH, F = p.F;

    if (tid == 0) {
        *abort_flag = 0;
        for (int s = 0; s < NSTAGE; ++s) {
            mbar_init(smem_u32(full + s), 1);
            mbar_init(smem_u32(empty + s), 1);
            mbar_init(smem_u32(full2 + s), NGW * 32);  // every lane of the gather warps arrives when its copies have landed
            mbar_init(smem_u32(empty2 + s), NCW);
        }
        mbar_init(smem_u32(acc_bar), 1);
        mbar_fence_init();
    }
    if (warp == NCW + 1) {  // the MMA warp owns the tensor memory
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *reinterpret_cast<volatile uint32_t*>(tmem_slot);

    int trace_ev = 0;
    auto mark = [&]() {
        if (p.trace && tid == 0 && trace_ev < 16) p.trace[static_cast<size_t>(cta) * 16 + trace_ev] = globaltimer_ns();
        ++trace_ev;
    };
    mark();
    unsigned bar_epoch = 0;
    // every thread of the CTA calls it; thread 0 counts in and spins (bounded) for the others
    auto grid_barrier = [&]() {
        tc_fence_before();
        __syncthreads();
        bar_epoch += 1;
        if (tid == 0) {
            const unsigned target = bar_epoch * static_cast<unsigned>(G);
            __threadfence();
            atomicAdd(p.sync, 1u);
            wait_bounded<96>([&] { return ld_acquire_u32(p.sync) >= target; }, ab, ST_TIMEOUT_GRID);
            __threadfence();
        }
        __syncthreads();
        tc_fence_after();
    };

    // ring cursors: each role keeps its own over the whole launch (GEMM: the TMA thread and the MMA thread;
    // attention: the gather warp and the consumer warps)
    Ring pr{smem_u32(ring), smem_u32(full), smem_u32(empty), 0, 0u};
    Ring cr = pr;
    Ring pr2{smem_u32(ring), smem_u32(full2), smem_u32(empty2), 0, 0u};
    Ring cr2 = pr2;
    uint32_t acc_phase = 0;

    // ---- one skinny GEMM phase: rows [ra0, ra1) of the weight matrix (and, with two = true, the same number
    // of rows from rb0: gate / up pairs) against the activations of all sequences over K columns.  All lanes
    // of warp 0 call epi(col0, v, u) for every group of 8 accumulator columns of the first range: v = the 8
    // values of this lane's sequence, u = the same columns of the second range (v again without one).
    auto gemm_phase = [&](const WMaps* wm, const CUtensorMap* am, int K, int ra0_in, int ra1_in, int rb0, bool two, auto epi) {
        // Narrow matrices (a few dozen rows per CTA) are bound by the NUMBER of MMAs, K / 16 per CTA whatever their
        // width: there the CTAs are grouped by ksplit, a group shares a row range ksplit times as long and each
        // member takes one slice of K; the partial outputs meet in global memory and, after a grid barrier, every
        // CTA adds the slices of its own (unsplit) rows in slice order and applies the epilogue.
        const int S = wm->ksplit > 1 ? wm->ksplit : 1;
        int ra0 = ra0_in, ra1 = ra1_in, blk0 = 0, nblk = K / 64, kslice = 0;
        if (S > 1) {
            const int rg = cta / S, NGR = G / S, NGt = p.H / 8;  // K-split projections all have H output rows
            kslice = cta - rg * S;
            ra0 = pbegin(rg, NGt, NGR) * 8;
            ra1 = pbegin(rg + 1, NGt, NGR) * 8;
            blk0 = pbegin(kslice, K / 64, S);
            nblk = pbegin(kslice + 1, K / 64, S) - blk0;
            if (rg >= NGR) ra1 = ra0;  // CTAs beyond the last whole group (none when ksplit divides the grid)
        }
        const int na = ra1 - ra0, NR = two ? 2 * na : na;
        const CUtensorMap* tw = (na == wm->rows_lo) ? &wm->lo : &wm->hi;
        const int kb = wm->kb, nset = wm->nset, set_stride = TMEM_COLS / nset;
        const int nst = (nblk + kb - 1) / kb;  // the last stage of a slice may hold fewer than kb of ITS blocks
        // Every CTA needs the same activation tiles; walking K in the same order they would all ask L2 for the
        // same lines at the same moment.  CTA c starts at stage c * nst / G of the K loop and wraps around, so
        // the CTAs are spread over the whole activation matrix (the sum order of a row is fixed by its CTA).
        const int rot = static_cast<int>((static_cast<long long>(cta) * nst) / G);
        if (na > 0) {
            if (warp == NCW && lane == 0) {
                // ---- TMA producer: one copy for the activations, one per weight range
                for (int s0 = 0; s0 < nst; ++s0) {
                    const int st = (s0 + rot) % nst;
                    mbar_wait(pr.empty + pr.stage * 8, pr.phase ^ 1u, ab, ST_TIMEOUT_EMPTY);
                    if (*ab.flag) break;
                    const uint32_t bar = pr.full + pr.stage * 8;
                    const uint32_t sb = pr.base + pr.stage * STAGE_BYTES;
                    mbar_arrive_expect_tx(bar, static_cast<uint32_t>(kb) * (A_KB_BYTES + NR * 128));
                    tma2d(sb, am, 0, (blk0 + st * kb) * 16, bar);
                    if (two) tma4d(sb + kb * A_KB_BYTES, tw, 0, ra0, 0, blk0 + st * kb, bar);  // [K block][gate rows | up rows]
                    else tma3d(sb + kb * A_KB_BYTES, tw, 0, ra0, blk0 + st * kb, bar);
                    pr.advance();
                }
            } else if (warp == NCW + 1 && lane == 0) {
                // ---- MMA issuer.  One thread feeds the tensor core, so the loop body is kept to a few
                // integer instructions per MMA (with descriptors rebuilt from scratch and a division per
                // step it measured 130 ns per MMA and bound the whole phase): the descriptors' constant
                // bits are formed once, per MMA only the 16-byte-unit start address is added.
                // Two weight ranges arrive K block by K block as [gate rows][up rows]: ONE B operand of 2 * na rows
                // (the host refuses more than 256 rows per CTA).
                const uint32_t idesc = idesc_f16(64, NR);
                const uint64_t desc_hi = smem_desc_sw128(0);       // everything but the start address
                const uint32_t setmask = static_cast<uint32_t>(nset - 1);  // nset is a power of two, at most 4 * kb
                const uint32_t a_kb = A_KB_BYTES >> 4, w_kb = static_cast<uint32_t>(NR * 128) >> 4;
                uint32_t nmma = 0;  // MMAs issued so far in this phase
                for (int s0 = 0; s0 < nst; ++s0) {
                    const int st = (s0 + rot) % nst;
                    const int jn = min(kb, nblk - st * kb);  // blocks of this stage that belong to this CTA's slice
                    mbar_wait(cr.full + cr.stage * 8, cr.phase, ab, ST_TIMEOUT_FULL);
                    if (*ab.flag) break;
                    tc_fence_after();
                    const uint32_t sb = cr.base + cr.stage * STAGE_BYTES;
                    uint32_t a_lo = sb >> 4, w_lo = (sb + kb * A_KB_BYTES) >> 4;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (j < jn) {
#pragma unroll
                            for (int k16 = 0; k16 < 4; ++k16) {
                                const uint32_t d0 = tmem_base + (nmma & setmask) * set_stride;
                                // the first MMA into each set overwrites, all later ones accumulate
                                const uint32_t accum = (nmma > setmask) ? 1u : 0u;
                                ++nmma;
                                const uint64_t adesc = desc_hi | (a_lo + 2u * k16);
                                umma_f16(d0, adesc, desc_hi | (w_lo + 2u * k16), idesc, accum);
                            }
                            a_lo += a_kb;
                            w_lo += w_kb;
                        }
                    }
                    umma_commit(cr.empty + cr.stage * 8);  // the stage is free once these MMAs have read it
                    cr.advance();
                }
                umma_commit(smem_u32(acc_bar));  // accumulators complete
            }
            if (warp == 0) {
                // ---- epilogue: thread = sequence (TMEM lane), 8 columns at a time, the sets added in order
                mbar_wait(smem_u32(acc_bar), acc_phase, ab, ST_TIMEOUT_FULL);
                tc_fence_after();
                if (!*ab.flag) {
                    for (int c0 = 0; c0 < na; c0 += 8) {
                        float v[8], u[8];
                        tmem_ld8(tmem_base + c0, v);
                        if (two) {
                            tmem_ld8(tmem_base + na + c0, u);
                        } else {
#pragma unroll
                            for (int k = 0; k < 8; ++k) u[k] = 0.f;
                        }
                        for (int q = 1; q < nset; ++q) {
                            float v2[8];
                            tmem_ld8(tmem_base + q * set_stride + c0, v2);
#pragma unroll
                            for (int k = 0; k < 8; ++k) v[k] += v2[k];
                            if (two) {
                                float u2[8];
                                tmem_ld8(tmem_base + q * set_stride + na + c0, u2);
#pragma unroll
                                for (int k = 0; k < 8; ++k) u[k] += u2[k];
                            }
                        }
                        if (S > 1) {
                            // this slice's share of the rows' dot products: added to the other slices' below
                            if (lane < B) {
                                float* dst = p.split32 + (static_cast<size_t>(kslice) * MAXB + lane) * p.H + ra0 + c0;
                                *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                                *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
                            }
                        } else {
                            epi(c0, v, u);
                        }
                    }
                }
                tc_fence_before();
            }
            acc_phase ^= 1u;
        }
        if (S > 1) {
            grid_barrier();
            // every CTA: its own rows of the unsplit partition, slices added in slice order
            if (warp == 0 && !*ab.flag) {
                for (int c0 = 0; c0 < ra1_in - ra0_in; c0 += 8) {
                    float v[8], u[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] = u[k] = 0.f;
                    if (lane < B) {
                        for (int q = 0; q < S; ++q) {
                            const float* src = p.split32 + (static_cast<size_t>(q) * MAXB + lane) * p.H + ra0_in + c0;
                            const float4 a = ld_cg_f32x4(src), b = ld_cg_f32x4(src + 4);
                            v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
                            v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
                        }
                    }
                    epi(c0, v, u);
                }
            }
        }
    };

    // ---- fused add + RMSNorm of every sequence: CTA b < B takes sequence b (consumer threads)
    auto norm_phase = [&]() {
        if (cta < B && tid < NCT) {
            const __half* x = p.input + static_cast<size_t>(cta) * H;
            const __half* r = p.residual ? p.residual + static_cast<size_t>(cta) * H : nullptr;
            __half* so = p.residual_out + static_cast<size_t>(cta) * H;
            float ss = 0.f;
            for (int v = tid; v < H / 8; v += NCT) {
                const uint4 xr = *reinterpret_cast<const uint4*>(x + v * 8);
                uint4 rr = make_uint4(0u, 0u, 0u, 0u);
                if (r) rr = *reinterpret_cast<const uint4*>(r + v * 8);
                const __half2* x2 = reinterpret_cast<const __half2*>(&xr);
                const __half2* r2 = reinterpret_cast<const __half2*>(&rr);
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 a = __half22float2(x2[k]), b = __half22float2(r2[k]);
                    o2[k] = __floats2half2_rn(a.x + b.x, a.y + b.y);
                    const float2 f = __half22float2(o2[k]);
                    ss = fmaf(f.x, f.x, ss);
                    ss = fmaf(f.y, f.y, ss);
                }
                *reinterpret_cast<uint4*>(so + v * 8) = o;
            }
            const float rstd = rsqrtf(csum(ss, red, tid) / static_cast<float>(H) + p.eps);
            for (int v = tid; v < H / 8; v += NCT) {
                // this thread re-reads what it wrote itself
                const uint4 sr = *reinterpret_cast<const uint4*>(so + v * 8);
                const uint4 gr = __ldg(reinterpret_cast<const uint4*>(p.norm_w + v * 8));
                const __half2* s2 = reinterpret_cast<const __half2*>(&sr);
                const __half2* g2 = reinterpret_cast<const __half2*>(&gr);
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 s = __half22float2(s2[k]), g = __half22float2(g2[k]);
                    o2[k] = __floats2half2_rn(s.x * rstd * g.x, s.y * rstd * g.y);
                }
                *reinterpret_cast<uint4*>(p.y16 + a_idx(cta, v * 8)) = o;
            }
        }
    };

    norm_phase();
    mark();
    grid_barrier();
    mark();

    if (p.mode == MODE_MLP) {
        // ---- gate / up rows in pairs, silu(gate) * up in the epilogue
        {
            const int NG = F / 8;
            const int g0 = pbegin(cta, NG, G) * 8, g1 = pbegin(cta + 1, NG, G) * 8, ng = g1 - g0;
            __half* mid = p.mid16;
            (void)ng;
            gemm_phase(&p.w_gu, &p.a_gu, H, g0, g1, F + g0, true, [&](int c0, const float (&gv)[8], const float (&uv)[8]) {
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float a0 = gv[2 * k] / (1.f + __expf(-gv[2 * k])) * uv[2 * k];
                    const float a1 = gv[2 * k + 1] / (1.f + __expf(-gv[2 * k + 1])) * uv[2 * k + 1];
                    o2[k] = __floats2half2_rn(a0, a1);
                }
                if (lane < B) *reinterpret_cast<uint4*>(mid + a_idx(lane, g0 + c0)) = o;
            });
        }
        mark();
        grid_barrier();
        mark();
        {
            const int NG = H / 8;
            const int r0 = pbegin(cta, NG, G) * 8, r1 = pbegin(cta + 1, NG, G) * 8;
            __half* out = p.output;
            gemm_phase(&p.w_down, &p.a_down, F, r0, r1, 0, false, [&](int c0, const float (&v)[8], const float (&)[8]) {
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int k = 0; k < 4; ++k) o2[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
                if (lane < B) *reinterpret_cast<uint4*>(out + static_cast<size_t>(lane) * H + r0 + c0) = o;
            });
        }
    } else {
        // ---- Q, K, V rows ([Q of all heads; K of all heads; V of all heads]) -> fp32 scratch
        {
            const int NG = 3 * H / 8;
            const int r0 = pbegin(cta, NG, G) * 8, r1 = pbegin(cta + 1, NG, G) * 8;
            float* qkv = p.qkv32;
            gemm_phase(&p.w_qkv, &p.a_qkv, H, r0, r1, 0, false, [&](int c0, const float (&v)[8], const float (&)[8]) {
                if (lane < B) {
                    float* dst = qkv + static_cast<size_t>(lane) * 3 * H + r0 + c0;
                    *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
                    *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
                }
            });
        }
        mark();
        grid_barrier();
        mark();

        // ---- attention over the cached rows: items (sequence, head, 128-row chunk), evenly split
        if (tid == 0) {
            int acc = 0;
            for (int b = 0; b < B; ++b) {
                const int s = max(0, __ldg(p.indptr + b + 1) - 1 - __ldg(p.indptr + b));
                pre[b] = acc;
                pre[MAXB + 1 + b] = s;
                acc += NH * ((s + KV_ROWS - 1) / KV_ROWS);
            }
            for (int b = B; b <= MAXB; ++b) pre[b] = acc;
        }
        __syncthreads();
        const int T = pre[B];
        const int ta = pbegin(cta, T, G), tb = pbegin(cta + 1, T, G);
        const __half* kpool = reinterpret_cast<const __half*>(__ldg(p.k_ptrs + p.layer_id));
        const __half* vpool = reinterpret_cast<const __half*>(__ldg(p.v_ptrs + p.layer_id));
        auto locate = [&](int t, int& b, int& h, int& ch, int& s) {
            b = 0;
            while (b + 1 < B && pre[b + 1] <= t) ++b;
            s = pre[MAXB + 1 + b];
            const int nch = (s + KV_ROWS - 1) / KV_ROWS;
            const int rem = t - pre[b];
            h = rem / nch;
            ch = rem - h * nch;
        };
        const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(D));
        if (warp >= NCW) {
            // ---- gather producers: NGW warps, each copies a quarter of a tile's rows with 16-byte asynchronous
            // copies (one bulk copy per row measured 8 us per item: the copy engine takes one operation at a
            // time; and one warp alone is bound by its own instruction stream at 4.6 us per item).  Lane l of
            // gather warp g fetches the pool index of row 32 g + l; the indices of the next item are requested
            // before the copies of the current one are issued.
            const int gw = warp - NCW;
            auto fetch_page = [&](int t, int& b, int& h, int& nvalid) {
                int ch, s;
                locate(t, b, h, ch, s);
                const int row0 = ch * KV_ROWS;
                nvalid = min(KV_ROWS, s - row0);
                const int r = gw * 32 + lane;
                return (r < nvalid) ? __ldg(p.indices + __ldg(p.indptr + b) + row0 + r) : 0;
            };
            int b = 0, h = 0, nvalid = 0, pg = 0;
            if (ta < tb) pg = fetch_page(ta, b, h, nvalid);
            for (int t = ta; t < tb; ++t) {
                int nb = 0, nh = 0, nnv = 0, npg = 0;
                if (t + 1 < tb) npg = fetch_page(t + 1, nb, nh, nnv);
#pragma unroll
                for (int kv = 0; kv < 2; ++kv) {
                    mbar_wait(pr2.empty + pr2.stage * 8, pr2.phase ^ 1u, ab, ST_TIMEOUT_EMPTY);
                    const uint32_t bar = pr2.full + pr2.stage * 8;
                    const uint32_t sb = pr2.base + pr2.stage * STAGE_BYTES;
                    const __half* pool = (kv ? vpool : kpool) + h * D;
                    // one warp instruction copies two rows: lanes 0-15 the 16-byte pieces of one row, lanes 16-31 of the next
                    const int hi = lane >> 4, piece = lane & 15;
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const int rl = 2 * i + hi;                 // row within this warp's quarter
                        const int page = __shfl_sync(0xffffffffu, pg, rl);
                        const int r = gw * 32 + rl;
                        if (r < nvalid) {
                            const __half* src = pool + static_cast<size_t>(page) * H + piece * 8;
                            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sb + r * D * 2 + piece * 16), "l"(src) : "memory");
                        }
                    }
                    // counts as this lane's arrival once its copies above are complete
                    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
                    pr2.advance();
                }
                b = nb, h = nh, nvalid = nnv, pg = npg;
            }
            asm volatile("cp.async.wait_all;" ::: "memory");
        } else if (tid < NCT) {
            // ---- consumers: 16 lanes per row, 8 rows per half-warp and tile, online softmax in fp32
            const int hw = lane >> 4, l16 = lane & 15;
            int cur_pair = -1;
            float qreg[8], acc[8], m_run = -INFINITY, l_run = 0.f;
            auto flush = [&](int pair) {
                const int slot = warp * 2 + hw;
#pragma unroll
                for (int k = 0; k < 8; ++k) mbuf[slot * D + l16 * 8 + k] = acc[k];
                if (l16 == 0) {
                    mlbuf[slot * 2] = m_run;
                    mlbuf[slot * 2 + 1] = l_run;
                }
                csync();
                float* dst = p.records + static_cast<size_t>(pair + cta) * REC;
                if (tid < D) {
                    float M = -INFINITY;
#pragma unroll
                    for (int i = 0; i < 16; ++i) M = fmaxf(M, mlbuf[i * 2]);
                    float a = 0.f, lsum = 0.f;
                    if (M > -INFINITY) {
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            const float w = exp2f(mlbuf[i * 2] - M);
                            a = fmaf(mbuf[i * D + tid], w, a);
                            lsum = fmaf(mlbuf[i * 2 + 1], w, lsum);
                        }
                    }
                    dst[tid] = a;
                    if (tid == 0) {
                        dst[D] = M;
                        dst[D + 1] = lsum;
                    }
                }
                csync();
            };
            for (int t = ta; t < tb; ++t) {
                int b, h, ch, s;
                locate(t, b, h, ch, s);
                const int pair = b * NH + h;
                if (pair != cur_pair) {
                    if (cur_pair >= 0) flush(cur_pair);
                    cur_pair = pair;
                    // rotated, scaled query of (b, h) into shared memory
                    if (tid < D) {
                        const float* qv = p.qkv32 + static_cast<size_t>(b) * 3 * H + h * D;
                        const float* cs = p.cos_sin + static_cast<size_t>(__ldg(p.positions + b)) * D;
                        const int d = tid, dh = d & 63;
                        const float c = __ldg(cs + dh), sn = __ldg(cs + 64 + dh);
                        const float self = __ldcg(qv + d), other = __ldcg(qv + (d < 64 ? d + 64 : d - 64));
                        q_s[d] = (d < 64 ? self * c - other * sn : self * c + other * sn) * qscale;
                    }
                    csync();
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        qreg[k] = q_s[l16 * 8 + k];
                        acc[k] = 0.f;
                    }
                    m_run = -INFINITY;
                    l_run = 0.f;
                }
                const int r0 = warp * 16 + hw * 8;
                const int grow = ch * KV_ROWS + r0;
                mbar_wait(cr2.full + cr2.stage * 8, cr2.phase, ab, ST_TIMEOUT_FULL);
                const __half* kt = reinterpret_cast<const __half*>(ring + static_cast<size_t>(cr2.stage) * STAGE_BYTES);
                float sc8[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float d = 0.f;
                    if (grow + j < s) {
                        const uint4 raw = *reinterpret_cast<const uint4*>(kt + (r0 + j) * D + l16 * 8);
                        const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const float2 f = __half22float2(h2[k]);
                            d = fmaf(f.x, qreg[2 * k], d);
                            d = fmaf(f.y, qreg[2 * k + 1], d);
                        }
                    }
                    sc8[j] = d;
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(cr2.empty + cr2.stage * 8);
                cr2.advance();
#pragma unroll
                for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) sc8[j] += __shfl_xor_sync(0xffffffffu, sc8[j], o);
                }
                float mx = m_run;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (grow + j >= s) sc8[j] = -INFINITY;
                    mx = fmaxf(mx, sc8[j]);
                }
                float scl = 1.f;
                if (mx > -INFINITY) {
                    scl = exp2f(m_run - mx);
                    m_run = mx;
#pragma unroll
                    for (int j = 0; j < 8; ++j) sc8[j] = (grow + j < s) ? exp2f(sc8[j] - mx) : 0.f;
                }
                mbar_wait(cr2.full + cr2.stage * 8, cr2.phase, ab, ST_TIMEOUT_FULL);
                const __half* vt = reinterpret_cast<const __half*>(ring + static_cast<size_t>(cr2.stage) * STAGE_BYTES);
                if (mx > -INFINITY) {
                    l_run *= scl;
#pragma unroll
                    for (int k = 0; k < 8; ++k) acc[k] *= scl;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        if (grow + j < s) {
                            const float pj = sc8[j];
                            l_run += pj;
                            const uint4 raw = *reinterpret_cast<const uint4*>(vt + (r0 + j) * D + l16 * 8);
                            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float2 f = __half22float2(h2[k]);
                                acc[2 * k] = fmaf(pj, f.x, acc[2 * k]);
                                acc[2 * k + 1] = fmaf(pj, f.y, acc[2 * k + 1]);
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(cr2.empty + cr2.stage * 8);
                cr2.advance();
            }
            if (cur_pair >= 0) flush(cur_pair);
        }
        mark();
        grid_barrier();
        mark();

        // ---- merge: pair (b, h) by CTA (pair % G): fold in the new token, append it to the pool
        if (tid < NCT) {
            for (int pair = cta; pair < B * NH; pair += G) {
                const int b = pair / NH, h = pair - b * NH;
                const int s = pre[MAXB + 1 + b];
                const int nch = (s + KV_ROWS - 1) / KV_ROWS;
                float qd = 0.f, kd = 0.f, vd = 0.f;
                if (tid < D) {
                    const float* base = p.qkv32 + static_cast<size_t>(b) * 3 * H + h * D;
                    const float* cs = p.cos_sin + static_cast<size_t>(__ldg(p.positions + b)) * D;
                    const int d = tid, dh = d & 63, dp = d < 64 ? d + 64 : d - 64;
                    const float c = __ldg(cs + dh), sn = __ldg(cs + 64 + dh);
                    const float q0 = __ldcg(base + d), q1 = __ldcg(base + dp);
                    const float k0 = __ldcg(base + H + d), k1 = __ldcg(base + H + dp);
                    qd = (d < 64 ? q0 * c - q1 * sn : q0 * c + q1 * sn) * qscale;
                    const __half k16 = __float2half_rn(d < 64 ? k0 * c - k1 * sn : k0 * c + k1 * sn);
                    const __half v16 = __float2half_rn(__ldcg(base + 2 * H + d));
                    kd = __half2float(k16);
                    vd = __half2float(v16);
                    // the slot of the new token: last entry of the sequence's page list
                    const int slot = __ldg(p.indices + __ldg(p.indptr + b + 1) - 1);
                    const size_t off = static_cast<size_t>(slot) * H + h * D + d;
                    const_cast<__half*>(reinterpret_cast<const __half*>(__ldg(p.k_ptrs + p.layer_id)))[off] = k16;
                    const_cast<__half*>(reinterpret_cast<const __half*>(__ldg(p.v_ptrs + p.layer_id)))[off] = v16;
                }
                const float s_new = csum(qd * kd, red, tid);
                if (tid < D) {
                    float M = s_new;
                    int c0 = 0, c1 = -1;
                    if (nch > 0) {
                        c0 = pof(pre[b] + h * nch, T, G);
                        c1 = pof(pre[b] + (h + 1) * nch - 1, T, G);
                    }
                    for (int c = c0; c <= c1; ++c)
                        if (pbegin(c + 1, T, G) > pbegin(c, T, G)) M = fmaxf(M, __ldcg(p.records + static_cast<size_t>(pair + c) * REC + D));
                    const float wn = exp2f(s_new - M);
                    float num = wn * vd, den = wn;
                    for (int c = c0; c <= c1; ++c) {
                        if (pbegin(c + 1, T, G) <= pbegin(c, T, G)) continue;
                        const float* rec = p.records + static_cast<size_t>(pair + c) * REC;
                        const float mj = __ldcg(rec + D);
                        if (mj > -INFINITY) {
                            const float w = exp2f(mj - M);
                            num = fmaf(w, __ldcg(rec + tid), num);
                            den = fmaf(w, __ldcg(rec + D + 1), den);
                        }
                    }
                    p.attn16[a_idx(b, h * D + tid)] = __float2half_rn(num / den);
                }
            }
        }
        mark();
        grid_barrier();
        mark();

        // ---- output projection
        {
            const int NG = H / 8;
            const int r0 = pbegin(cta, NG, G) * 8, r1 = pbegin(cta + 1, NG, G) * 8;
            __half* out = p.output;
            gemm_phase(&p.w_o, &p.a_o, H, r0, r1, 0, false, [&](int c0, const float (&v)[8], const float (&)[8]) {
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int k = 0; k < 4; ++k) o2[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
                if (lane < B) *reinterpret_cast<uint4*>(out + static_cast<size_t>(lane) * H + r0 + c0) = o;
            });
        }
    }

    // ---- leave: tensor memory back, exit count, the last CTA re-arms the barrier words
    tc_fence_before();
    __syncthreads();
    mark();
    if (warp == NCW + 1) tmem_dealloc(tmem_base, TMEM_COLS);
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(p.sync + 1, 1u);
        if (old == static_cast<unsigned>(G) - 1u) {
            p.sync[0] = 0u;
            p.sync[1] = 0u;
            __threadfence();
        }
    }
}

__host__ __device__ inline size_t smem_bytes() {
    return static_cast<size_t>(NSTAGE) * STAGE_BYTES + (D + 16 * D + 32 + 32) * 4 + (2 * MAXB + 2) * 4 + (4 * NSTAGE + 1) * 8 + 16;
}

}  // namespace lb
}  // namespace cfb
