// Host side of the batched Llama decode blocks (llama_batch_kernel.cuh): argument checks, tensor maps
// (encoded on the host and passed to the kernel as launch parameters, like the reference does in
// include/5090/llama/llama_kernel_batch_sglang_dispatch.cu:46-84, but cached per weight tensor), the
// per-device scratch and the cooperative launch.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <tuple>

#include "../../include/clusterfusion_b200.h"
#include "host_common.h"
#include "llama_batch_kernel.cuh"

using namespace cfb;

namespace {

struct LbDevice {
    bool ready = false;
    int sm_count = 0;
    char* base = nullptr;
    __half *y16 = nullptr, *attn16 = nullptr, *mid16 = nullptr;
    float *qkv32 = nullptr, *records = nullptr, *split32 = nullptr;
    unsigned* sync = nullptr;
    int* status = nullptr;
    std::map<std::tuple<const void*, int64_t, int64_t, int>, lb::WMaps> wmaps;   // (weights, rows, cols, ranges per CTA)
    std::map<std::tuple<const void*, int64_t, int>, CUtensorMap> amaps;           // (activations, columns, K blocks per stage)
    unsigned long long* trace = nullptr;   // diagnostics
};

constexpr int LB_MAX_DEVICES = 64;
constexpr int LB_H = 4096, LB_NH = 32;      // include/5090/llama/config.h:1-4 of the reference
constexpr int LB_MAX_F = 16384;
constexpr int LB_MAX_GRID = 256;
constexpr int LB_MAX_KSPLIT = 4;   // K slices of a narrow projection (groups of CTAs share a row range)
LbDevice g_lb[LB_MAX_DEVICES];
std::mutex g_lb_mu;

// 128-byte-swizzled fp16 tensor map of `rank` dimensions (innermost first; strides in bytes for dimensions 1..)
int encode_sw128(CUtensorMap* tm, const void* ptr, int rank, const cuuint64_t* dims, const cuuint64_t* strides,
                 const cuuint32_t* box) {
    CfEncodeTiledFn enc = cf_host_encode_fn();
    if (!enc) return cf_host_fail(CF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return cf_host_fail(CF_ERR_INVALID, "tensor base not 16-byte aligned");
    cuuint32_t es[4] = {1, 1, 1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(ptr), dims, strides,
                     box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cf_host_fail(CF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return CF_OK;
}

#define LB_CUDA(expr)                                                                                        \
    do {                                                                                                     \
        cudaError_t e_ = (expr);                                                                             \
        if (e_ != cudaSuccess) return cf_host_fail(CF_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

size_t up256(size_t v) { return (v + 255) / 256 * 256; }

int lb_device(cudaStream_t st, LbDevice** out) {
    int dev = -1;
    LB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= LB_MAX_DEVICES) return cf_host_fail(CF_ERR_UNSUPPORTED, "device index %d", dev);
    LbDevice& d = g_lb[dev];
    if (!d.ready) {
        int rc = cf_host_refuse_in_capture(st, "first batched Llama call on a device (it allocates the scratch)");
        if (rc) return rc;
        cudaDeviceProp prop;
        LB_CUDA(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return cf_host_fail(CF_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                                prop.major, prop.minor);
        d.sm_count = prop.multiProcessorCount;
        if (d.sm_count > LB_MAX_GRID) return cf_host_fail(CF_ERR_UNSUPPORTED, "%d SMs", d.sm_count);
        const size_t o_y = 0, o_attn = o_y + up256(sizeof(__half) * 16 * LB_H), o_mid = o_attn + up256(sizeof(__half) * 16 * LB_H);
        const size_t o_qkv = o_mid + up256(sizeof(__half) * 16 * LB_MAX_F);
        const size_t o_rec = o_qkv + up256(sizeof(float) * 16 * 3 * LB_H);
        const size_t o_split = o_rec + up256(sizeof(float) * (16 * LB_NH + LB_MAX_GRID) * lb::REC);
        const size_t o_sync = o_split + up256(sizeof(float) * LB_MAX_KSPLIT * 16 * LB_H);
        const size_t total = o_sync + 256;
        LB_CUDA(cudaMalloc(&d.base, total));
        LB_CUDA(cudaMemset(d.base, 0, total));
        d.y16 = reinterpret_cast<__half*>(d.base + o_y);
        d.attn16 = reinterpret_cast<__half*>(d.base + o_attn);
        d.mid16 = reinterpret_cast<__half*>(d.base + o_mid);
        d.qkv32 = reinterpret_cast<float*>(d.base + o_qkv);
        d.records = reinterpret_cast<float*>(d.base + o_rec);
        d.split32 = reinterpret_cast<float*>(d.base + o_split);
        d.sync = reinterpret_cast<unsigned*>(d.base + o_sync);
        d.status = reinterpret_cast<int*>(d.base + o_sync + 16);
        LB_CUDA(cudaFuncSetAttribute(lb::llama_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(lb::smem_bytes())));
        int nb = 0;
        LB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, lb::llama_batch_kernel, lb::THREADS, lb::smem_bytes()));
        if (nb < 1) return cf_host_fail(CF_ERR_UNSUPPORTED, "the batched kernel does not fit on an SM of this device");
        d.ready = true;
    }
    *out = &d;
    return CF_OK;
}

// Tensor maps and stage geometry of one weight matrix [rows, cols] whose rows are split over `grid` CTAs in 8-row
// granules, `ranges` row ranges per CTA (2: the gate / up halves of a merged matrix, rows = rows of one half).
int weight_maps(LbDevice& d, const void* w, int64_t rows, int64_t cols, int ranges, lb::WMaps* out) {
    if (ranges != 1 && ranges != 2) return cf_host_fail(CF_ERR_INVALID, "%d row ranges per CTA", ranges);
    // Narrow matrices -- fewer than 40 rows per CTA -- are cut along K as well: groups of ksplit CTAs share a row
    // range ksplit times as long (K / 16 MMAs per CTA whatever their width is what bounds such a projection).
    // Only for matrices with H output rows (the scratch and the kernel's regrouping assume it).
    int ksplit = 1;
    {
        const char* e = getenv("CFB200_LB_KSPLIT");
        const int want = e ? atoi(e) : LB_MAX_KSPLIT;
        if (ranges == 1 && rows == LB_H && rows / d.sm_count < 40 && want > 1 && want <= LB_MAX_KSPLIT &&
            d.sm_count % want == 0 && (cols / 64) >= 4 * want)
            ksplit = want;
    }
    const int ngroups = d.sm_count / ksplit;
    auto key = std::make_tuple(w, rows, cols, ranges * 16 + ksplit);
    auto it = d.wmaps.find(key);
    if (it == d.wmaps.end()) {
        if (d.wmaps.size() >= 4096) d.wmaps.clear();  // maps are host objects: nothing in flight refers to them
        lb::WMaps m;
        memset(&m, 0, sizeof(m));
        const int64_t ng = rows / 8;
        m.rows_lo = static_cast<int>(ng / ngroups) * 8;
        m.ksplit = ksplit;
        const int nr_max = ranges * (m.rows_lo + 8);
        if (nr_max > 256) return cf_host_fail(CF_ERR_UNSUPPORTED, "%d weight rows per CTA (at most 256)", nr_max);
        const int nkb = static_cast<int>(cols / 64);
        int kb = 4;
        // (an unsplit K must be a whole number of stages; a slice's last stage may be ragged)
        while (kb > 1 && (kb * (lb::A_KB_BYTES + nr_max * 128) > lb::STAGE_BYTES || (ksplit == 1 && (nkb % kb) != 0))) kb >>= 1;
        if (kb * (lb::A_KB_BYTES + nr_max * 128) > lb::STAGE_BYTES)
            return cf_host_fail(CF_ERR_UNSUPPORTED, "a ring stage cannot hold %d weight rows", nr_max);
        m.kb = kb;
        // Accumulator sets: consecutive MMAs go to different sets of tensor-memory columns, so that each is an
        // independent chain (an MMA of this size is latency-, not throughput-bound).  As many as fit: a set is
        // 512 / nset columns wide and must hold the CTA's rows; every set must be written in every stage
        // (4 MMAs per K block); a power of two.  CFB200_LB_NSET caps it (experiments).
        {
            int cap = 512 / nr_max;
            if (cap > 4 * kb) cap = 4 * kb;
            if (cap > 16) cap = 16;
            const char* e = getenv("CFB200_LB_NSET");
            if (e && atoi(e) > 0 && atoi(e) < cap) cap = atoi(e);
            m.nset = 1;
            while (2 * m.nset <= cap) m.nset *= 2;
        }
        // {64 K elements, rows, K / 64 blocks}: strides of dimension 1 (a row) and 2 (the next 64 columns).  With
        // two ranges (the gate and up halves of a merged matrix) the half is a dimension of its own between
        // them, {64, rows, 2, K / 64}: ONE copy then brings, K block by K block, the CTA's gate rows followed
        // by its up rows -- a single B operand of 2 r rows for the tensor core.
        for (int v = 0; v < 2; ++v) {
            const int r = m.rows_lo + 8 * v;
            if (r == 0) continue;  // never used: every CTA then holds rows_lo + 8 rows or none
            int rc;
            if (ranges == 2) {
                cuuint64_t dims[4] = {64, static_cast<cuuint64_t>(rows), 2, static_cast<cuuint64_t>(nkb)};
                cuuint64_t strides[3] = {static_cast<cuuint64_t>(cols) * 2, static_cast<cuuint64_t>(rows) * cols * 2, 128};
                cuuint32_t box[4] = {64, static_cast<cuuint32_t>(r), 2, static_cast<cuuint32_t>(kb)};
                rc = encode_sw128(v ? &m.hi : &m.lo, w, 4, dims, strides, box);
            } else {
                cuuint64_t dims[3] = {64, static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(nkb)};
                cuuint64_t strides[2] = {static_cast<cuuint64_t>(cols) * 2, 128};
                cuuint32_t box[3] = {64, static_cast<cuuint32_t>(r), static_cast<cuuint32_t>(kb)};
                rc = encode_sw128(v ? &m.hi : &m.lo, w, 3, dims, strides, box);
            }
            if (rc) return rc;
        }
        it = d.wmaps.emplace(key, m).first;
    }
    *out = it->second;
    return CF_OK;
}

// K-block-major activations [cols / 64][16][64]: {64, 16 * cols / 64} with box {64, 16 * kb}
int act_map(LbDevice& d, const void* a, int64_t cols, int kb, CUtensorMap* out) {
    auto key = std::make_tuple(a, cols, kb);
    auto it = d.amaps.find(key);
    if (it == d.amaps.end()) {
        CUtensorMap m;
        cuuint64_t dims[2] = {64, static_cast<cuuint64_t>(16 * (cols / 64))};
        cuuint64_t strides[1] = {128};
        cuuint32_t box[2] = {64, static_cast<cuuint32_t>(16 * kb)};
        int rc = encode_sw128(&m, a, 2, dims, strides, box);
        if (rc) return rc;
        it = d.amaps.emplace(key, m).first;
    }
    *out = it->second;
    return CF_OK;
}

int launch_lb(LbDevice& d, lb::Params& p, cudaStream_t st) {
    p.y16 = d.y16;
    p.attn16 = d.attn16;
    p.mid16 = d.mid16;
    p.qkv32 = d.qkv32;
    p.split32 = d.split32;
    p.records = d.records;
    p.sync = d.sync;
    p.status = d.status;
    p.trace = d.trace;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(d.sm_count);
    lc.blockDim = dim3(lb::THREADS);
    lc.dynamicSmemBytes = lb::smem_bytes();
    lc.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;  // the phases meet at grid barriers: all CTAs must be resident
    at[0].val.cooperative = 1;
    lc.attrs = at;
    // CFB200_COOPERATIVE=0 (profilers): a plain launch; one CTA per SM is resident anyway when nothing else runs
    static const bool coop = [] { const char* e = getenv("CFB200_COOPERATIVE"); return !(e && e[0] == '0'); }();
    lc.numAttrs = coop ? 1 : 0;
    void* args[1] = {&p};
    cudaError_t e = cudaLaunchKernelExC(&lc, reinterpret_cast<const void*>(&lb::llama_batch_kernel), args);
    if (e != cudaSuccess)
        return cf_host_fail(CF_ERR_CUDA, "batched Llama launch failed: %s (grid %d, smem %zu)", cudaGetErrorString(e), d.sm_count,
                            lb::smem_bytes());
    return CF_OK;
}

}  // namespace

// device status word of the batched path on the current device (0 when it was never used); clears it
int cf_host_lb_probe_status(int dev, int* status) {
    *status = 0;
    std::lock_guard<std::mutex> lk(g_lb_mu);
    if (dev < 0 || dev >= LB_MAX_DEVICES || !g_lb[dev].ready) return CF_OK;
    int s = 0;
    LB_CUDA(cudaMemcpy(&s, g_lb[dev].status, sizeof(int), cudaMemcpyDeviceToHost));
    if (s != 0) {
        LB_CUDA(cudaMemset(g_lb[dev].status, 0, sizeof(int)));
        LB_CUDA(cudaMemset(g_lb[dev].sync, 0, 2 * sizeof(unsigned)));
    }
    *status = s;
    return CF_OK;
}

extern "C" {

int cf_debug_set_llama_batch_trace(void* device_buffer, int64_t n_slots) {
    int dev = -1;
    LB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= LB_MAX_DEVICES) return cf_host_fail(CF_ERR_UNSUPPORTED, "device index %d", dev);
    if (device_buffer && n_slots < static_cast<int64_t>(LB_MAX_GRID) * 16)
        return cf_host_fail(CF_ERR_INVALID, "the timeline buffer needs %d slots", LB_MAX_GRID * 16);
    std::lock_guard<std::mutex> lk(g_lb_mu);
    g_lb[dev].trace = static_cast<unsigned long long*>(device_buffer);
    return CF_OK;
}

int cf_llama_decoder_layer_batch_sglang(void* output, void* residual_output, const void* input, const void* residual,
                                        const void* weight_qkv, const void* weight_o, const int* paged_kv_indptr,
                                        const int* paged_kv_indices, const uint64_t* k_cache_ptrs,
                                        const uint64_t* v_cache_ptrs, int layer_id, const void* rms_input_weight, float eps,
                                        const int64_t* positions, const float* cos_sin, int64_t batch, void* stream) {
    if (!output || !residual_output || !input || !weight_qkv || !weight_o || !paged_kv_indptr || !paged_kv_indices ||
        !k_cache_ptrs || !v_cache_ptrs || !rms_input_weight || !positions || !cos_sin)
        return cf_host_fail(CF_ERR_INVALID, "null pointer");
    if (batch < 1 || batch > lb::MAXB) return cf_host_fail(CF_ERR_UNSUPPORTED, "batch %lld (1..%d)", (long long)batch, lb::MAXB);
    if (layer_id < 0) return cf_host_fail(CF_ERR_INVALID, "layer_id %d", layer_id);
    if (residual && residual == residual_output) return cf_host_fail(CF_ERR_INVALID, "residual_output must not alias residual");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> lk(g_lb_mu);
    LbDevice* d;
    int rc = lb_device(st, &d);
    if (rc) return rc;
    lb::Params p;
    memset(&p, 0, sizeof(p));
    if ((rc = weight_maps(*d, weight_qkv, 3 * LB_H, LB_H, 1, &p.w_qkv))) return rc;
    if ((rc = weight_maps(*d, weight_o, LB_H, LB_H, 1, &p.w_o))) return rc;
    if ((rc = act_map(*d, d->y16, LB_H, p.w_qkv.kb, &p.a_qkv))) return rc;
    if ((rc = act_map(*d, d->attn16, LB_H, p.w_o.kb, &p.a_o))) return rc;
    p.mode = lb::MODE_ATTN;
    p.B = static_cast<int>(batch);
    p.H = LB_H;
    p.NH = LB_NH;
    p.F = 0;
    p.eps = eps;
    p.input = static_cast<const __half*>(input);
    p.residual = static_cast<const __half*>(residual);
    p.norm_w = static_cast<const __half*>(rms_input_weight);
    p.residual_out = static_cast<__half*>(residual_output);
    p.output = static_cast<__half*>(output);
    p.indptr = paged_kv_indptr;
    p.indices = paged_kv_indices;
    p.k_ptrs = reinterpret_cast<const unsigned long long*>(k_cache_ptrs);
    p.v_ptrs = reinterpret_cast<const unsigned long long*>(v_cache_ptrs);
    p.layer_id = layer_id;
    p.positions = reinterpret_cast<const long long*>(positions);
    p.cos_sin = cos_sin;
    return launch_lb(*d, p, st);
}

int cf_llama_mlp_batch_sglang(const void* input, const void* residual, const void* gate_up_weight, const void* down_weight,
                              const void* rms_weight, float eps, int64_t ffn, int64_t batch, void* output,
                              void* residual_out, void* stream) {
    if (!input || !gate_up_weight || !down_weight || !rms_weight || !output || !residual_out)
        return cf_host_fail(CF_ERR_INVALID, "null pointer");
    if (batch < 1 || batch > lb::MAXB) return cf_host_fail(CF_ERR_UNSUPPORTED, "batch %lld (1..%d)", (long long)batch, lb::MAXB);
    if (residual && residual == residual_out) return cf_host_fail(CF_ERR_INVALID, "residual_out must not alias residual");
    if (ffn <= 0 || (ffn % 64) != 0 || ffn > LB_MAX_F)
        return cf_host_fail(CF_ERR_INVALID, "ffn %lld must be a positive multiple of 64 and at most %d", (long long)ffn, LB_MAX_F);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    std::lock_guard<std::mutex> lk(g_lb_mu);
    LbDevice* d;
    int rc = lb_device(st, &d);
    if (rc) return rc;
    lb::Params p;
    memset(&p, 0, sizeof(p));
    if ((rc = weight_maps(*d, gate_up_weight, ffn, LB_H, 2, &p.w_gu))) return rc;
    if ((rc = weight_maps(*d, down_weight, LB_H, ffn, 1, &p.w_down))) return rc;
    if ((rc = act_map(*d, d->y16, LB_H, p.w_gu.kb, &p.a_gu))) return rc;
    if ((rc = act_map(*d, d->mid16, ffn, p.w_down.kb, &p.a_down))) return rc;
    p.mode = lb::MODE_MLP;
    p.B = static_cast<int>(batch);
    p.H = LB_H;
    p.NH = LB_NH;
    p.F = static_cast<int>(ffn);
    p.eps = eps;
    p.input = static_cast<const __half*>(input);
    p.residual = static_cast<const __half*>(residual);
    p.norm_w = static_cast<const __half*>(rms_weight);
    p.residual_out = static_cast<__half*>(residual_out);
    p.output = static_cast<__half*>(output);
    return launch_lb(*d, p, st);
}

}  // extern "C"
