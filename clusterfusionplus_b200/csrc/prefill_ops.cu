// Prompt ingestion, the parts around the GEMMs: both LayerNorms of a GPT-NeoX block in one pass over the hidden
// states, and the split of the fused QKV projection into rotated queries, rotated keys (written to their cache
// rows) and values (written to theirs).  HBM-bound elementwise kernels for sm_100a; every position is a row.
// The reference has no prefill (tests/benchmark_full.py:195-199 runs the prompt through the HuggingFace model);
// the arithmetic follows its decode kernel: LayerNorm with eps 1e-5 in fp32 (include/5090/pythia_6b9/kernel.cuh
// :130-200), rotate-half RoPE on the first `rotary` dims of every head (:300-360), fp16 storage.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/clusterfusion_b200.h"
#include "host_common.h"

namespace {

constexpr int LN_THREADS = 256;
constexpr int LN_MAX_VEC = 4;  // 8-element vectors per thread: hidden up to 256 * 4 * 8 = 8192

__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
    __syncthreads();  // red[] may still be read from the previous call
    if (l == 0) red[w] = v;
    __syncthreads();
    float t = (l < LN_THREADS / 32) ? red[l] : 0.f;
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    return __shfl_sync(0xffffffffu, t, 0);
}

// one CTA per row: y1 = LN(x; g1, b1), y2 = LN(x; g2, b2); mean and variance (two-pass, fp32) are shared
__global__ void __launch_bounds__(LN_THREADS) prefill_layernorm2_kernel(const __half* __restrict__ x, const __half* __restrict__ g1,
                                                                         const __half* __restrict__ b1, const __half* __restrict__ g2,
                                                                         const __half* __restrict__ b2, __half* __restrict__ y1,
                                                                         __half* __restrict__ y2, int H, float eps) {
    __shared__ float red[LN_THREADS / 32];
    const size_t row = blockIdx.x;
    const int nvec = H >> 3;
    float xv[LN_MAX_VEC][8];
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < LN_MAX_VEC; ++j) {
        const int v = j * LN_THREADS + threadIdx.x;
        if (v < nvec) {
            const uint4 raw = __ldg(reinterpret_cast<const uint4*>(x + row * H) + v);
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(h2[k]);
                xv[j][2 * k] = f.x;
                xv[j][2 * k + 1] = f.y;
                s += f.x + f.y;
            }
        }
    }
    const float mean = block_sum_256(s, red) / static_cast<float>(H);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < LN_MAX_VEC; ++j) {
        const int v = j * LN_THREADS + threadIdx.x;
        if (v < nvec) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float d = xv[j][k] - mean;
                ss = fmaf(d, d, ss);
            }
        }
    }
    const float rstd = rsqrtf(block_sum_256(ss, red) / static_cast<float>(H) + eps);
#pragma unroll
    for (int j = 0; j < LN_MAX_VEC; ++j) {
        const int v = j * LN_THREADS + threadIdx.x;
        if (v < nvec) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                const __half* g = which ? g2 : g1;
                const __half* b = which ? b2 : b1;
                __half* y = which ? y2 : y1;
                if (!y) continue;
                const uint4 graw = __ldg(reinterpret_cast<const uint4*>(g) + v);
                const uint4 braw = __ldg(reinterpret_cast<const uint4*>(b) + v);
                const __half2* gg = reinterpret_cast<const __half2*>(&graw);
                const __half2* bb = reinterpret_cast<const __half2*>(&braw);
                uint4 o;
                __half2* o2 = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 gf = __half22float2(gg[k]), bf = __half22float2(bb[k]);
                    o2[k] = __floats2half2_rn((xv[j][2 * k] - mean) * rstd * gf.x + bf.x,
                                              (xv[j][2 * k + 1] - mean) * rstd * gf.y + bf.y);
                }
                reinterpret_cast<uint4*>(y + row * H)[v] = o;
            }
        }
    }
}

// qkv [m][heads][3][D] (the fused projection's row order: per head q, k, v) -> q_out [m][heads][D] rotated,
// k_rows [m][heads * D] rotated, v_rows [m][heads * D]; position of row i is i (a prompt starts at 0);
// cos / sin [m][rotary] fp32.  One CTA per position, one thread per pair of elements.
__global__ void __launch_bounds__(256) prefill_rope_split_kernel(const __half* __restrict__ qkv, const float* __restrict__ cos,
                                                                  const float* __restrict__ sin, __half* __restrict__ q_out,
                                                                  __half* __restrict__ k_rows, __half* __restrict__ v_rows, int heads,
                                                                  int D, int R, size_t kv_stride) {
    const size_t pos = blockIdx.x;
    const int half_r = R >> 1;
    const int per_head = D >> 1;  // element pairs (2e, 2e + 1) of one vector
    const __half* src = qkv + pos * static_cast<size_t>(heads) * 3 * D;
    const float* cr = cos + pos * R;
    const float* sr = sin + pos * R;
    for (int t = threadIdx.x; t < heads * 3 * per_head; t += blockDim.x) {
        const int h = t / (3 * per_head), rem = t - h * 3 * per_head;
        const int part = rem / per_head, e = (rem - part * per_head) * 2;
        const __half* vsrc = src + (static_cast<size_t>(h) * 3 + part) * D;
        float2 val = __half22float2(*reinterpret_cast<const __half2*>(vsrc + e));
        if (part < 2 && e < R) {
            // rotate-half: out[d] = x[d] cos[d] + (d < R/2 ? -x[d + R/2] : x[d - R/2]) sin[d]
            const int pe = (e < half_r) ? e + half_r : e - half_r;
            const float2 pv = __half22float2(*reinterpret_cast<const __half2*>(vsrc + pe));
            const float sg = (e < half_r) ? -1.f : 1.f;
            val.x = val.x * cr[e] + sg * pv.x * sr[e];
            val.y = val.y * cr[e + 1] + sg * pv.y * sr[e + 1];
        }
        const __half2 o = __floats2half2_rn(val.x, val.y);
        if (part == 0) *reinterpret_cast<__half2*>(q_out + (pos * heads + h) * D + e) = o;
        else if (part == 1) *reinterpret_cast<__half2*>(k_rows + pos * kv_stride + static_cast<size_t>(h) * D + e) = o;
        else *reinterpret_cast<__half2*>(v_rows + pos * kv_stride + static_cast<size_t>(h) * D + e) = o;
    }
}

}  // namespace

extern "C" {

int cf_prefill_layernorm2(const void* x, const void* gamma1, const void* beta1, const void* gamma2, const void* beta2,
                          void* y1, void* y2, int64_t m, int64_t hidden, float eps, void* stream) {
    if (!x || !gamma1 || !beta1 || !y1) return cf_host_fail(CF_ERR_INVALID, "null pointer");
    if (y2 && (!gamma2 || !beta2)) return cf_host_fail(CF_ERR_INVALID, "second output without its weight and bias");
    if (m < 1 || m > 0x7fffffff) return cf_host_fail(CF_ERR_INVALID, "rows %lld", (long long)m);
    if (hidden < 8 || (hidden % 8) != 0 || hidden > LN_THREADS * LN_MAX_VEC * 8)
        return cf_host_fail(CF_ERR_INVALID, "hidden %lld must be a multiple of 8, at most %d", (long long)hidden,
                            LN_THREADS * LN_MAX_VEC * 8);
    prefill_layernorm2_kernel<<<static_cast<unsigned>(m), LN_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<const __half*>(gamma1), static_cast<const __half*>(beta1),
        static_cast<const __half*>(gamma2), static_cast<const __half*>(beta2), static_cast<__half*>(y1),
        static_cast<__half*>(y2), static_cast<int>(hidden), eps);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cf_host_fail(CF_ERR_CUDA, "prefill LayerNorm launch failed: %s", cudaGetErrorString(e));
    return CF_OK;
}

int cf_prefill_rope_split(const void* qkv, const float* cos, const float* sin, void* q_out, void* k_rows, void* v_rows,
                          int64_t m, int64_t heads, int64_t head_dim, int64_t rotary, int64_t kv_row_stride, void* stream) {
    if (!qkv || !cos || !sin || !q_out || !k_rows || !v_rows) return cf_host_fail(CF_ERR_INVALID, "null pointer");
    if (m < 1 || m > 0x7fffffff) return cf_host_fail(CF_ERR_INVALID, "rows %lld", (long long)m);
    if (heads < 1 || head_dim < 2 || (head_dim & 1) || rotary < 0 || rotary > head_dim || (rotary & 3))
        return cf_host_fail(CF_ERR_INVALID, "heads %lld, head_dim %lld, rotary %lld (rotary a multiple of 4)", (long long)heads,
                            (long long)head_dim, (long long)rotary);
    if (kv_row_stride < heads * head_dim) return cf_host_fail(CF_ERR_INVALID, "cache row stride %lld", (long long)kv_row_stride);
    prefill_rope_split_kernel<<<static_cast<unsigned>(m), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(qkv), cos, sin, static_cast<__half*>(q_out), static_cast<__half*>(k_rows),
        static_cast<__half*>(v_rows), static_cast<int>(heads), static_cast<int>(head_dim), static_cast<int>(rotary),
        static_cast<size_t>(kv_row_stride));
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return cf_host_fail(CF_ERR_CUDA, "prefill RoPE launch failed: %s", cudaGetErrorString(e));
    return CF_OK;
}

}  // extern "C"
