// C-ABI host side of the fused decode path: argument checks, tensor-map cache,
// launch geometry, per-layer contexts and the whole-model decoder.  No torch
// types, no CPU compute path: without a CUDA device every entry point fails.
//
// Host-side counterpart of the reference's dispatchers
// (include/5090/pythia_6b9/pythia_kernel_dispatch.cu, ..._graph.cu,
// include/5090/pythia_2b8/pythia_kernel_dispatch_split.cu), which rebuild six
// tensor maps, allocate five tensors and synchronise the device twice on every
// call; here descriptors are built once and cached, outputs belong to the caller
// (or to a context) and nothing synchronises.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/clusterfusion_b200.h"
#include "decode_kernel.cuh"
#include "host_common.h"
#include "prefill_gemm.h"

using namespace cfb;

namespace {

thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}

#define CF_CUDA(expr)                                                                              \
    do {                                                                                           \
        cudaError_t e_ = (expr);                                                                   \
        if (e_ != cudaSuccess) return fail(CF_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

// A descriptor upload copies from host memory that does not outlive the call.  Recorded into a
// stream capture, the copy node would keep that pointer and read it again at every replay, so an
// upload is refused while the stream is capturing: the caller makes the call once outside the
// capture (which caches the descriptor) and captures afterwards.
int refuse_upload_in_capture(cudaStream_t st, const char* what) {
    cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
    cudaError_t e = cudaStreamIsCapturing(st, &cs);
    if (e != cudaSuccess) return fail(CF_ERR_CUDA, "cudaStreamIsCapturing failed: %s", cudaGetErrorString(e));
    if (cs != cudaStreamCaptureStatusNone)
        return fail(CF_ERR_INVALID,
                    "%s: these tensors need a descriptor upload, which cannot be recorded into a stream capture; "
                    "call once with the same tensors outside the capture first",
                    what);
    return CF_OK;
}

const CfDims kDims[2] = {
    {2560, 32, 80, 20, 10240, 50304},
    {4096, 32, 128, 32, 16384, 50432},
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// fp16 row-major [outer, inner] with `row_stride` elements between rows
int encode_2d(CUtensorMap* tm, const void* ptr, uint64_t inner, uint64_t outer, uint64_t row_stride,
              uint32_t box_inner, uint32_t box_outer,
              CUtensorMapL2promotion promo = CU_TENSOR_MAP_L2_PROMOTION_L2_256B) {
    EncodeTiledFn enc = get_encode();
    if (!enc) return fail(CF_ERR_CUDA, "cuTensorMapEncodeTiled entry point not available");
    if ((reinterpret_cast<uintptr_t>(ptr) & 15) != 0) return fail(CF_ERR_INVALID, "tensor base not 16-byte aligned");
    if ((row_stride * 2) % 16 != 0) return fail(CF_ERR_INVALID, "row stride not a multiple of 16 bytes");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {row_stride * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t es[2] = {1, 1};
    CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, es,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, promo, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return CF_OK;
}

// contiguous row-major weight [rows, cols]: boxes of 8, 16, 24, 32 and 64 rows x 256 columns
int encode_weight(WeightMaps* m, const void* ptr, uint64_t cols, uint64_t rows) {
    int rc;
    if ((rc = encode_2d(&m->r8, ptr, cols, rows, cols, KCHUNK, GRAN))) return rc;
    if ((rc = encode_2d(&m->r16, ptr, cols, rows, cols, KCHUNK, 2 * GRAN))) return rc;
    if ((rc = encode_2d(&m->r24, ptr, cols, rows, cols, KCHUNK, 3 * GRAN))) return rc;
    if ((rc = encode_2d(&m->r32, ptr, cols, rows, cols, KCHUNK, 4 * GRAN))) return rc;
    return encode_2d(&m->r64, ptr, cols, rows, cols, KCHUNK, 8 * GRAN);
}

struct Workspace {
    void* base = nullptr;
    uint2* qkv_ll = nullptr;
    uint2* hid_ll[2] = {nullptr, nullptr};
    float *mid_f32 = nullptr, *attn_part = nullptr, *attn_new = nullptr, *amax_val = nullptr;
    int* amax_idx = nullptr;
    unsigned* sync = nullptr;
    int* status = nullptr;
};

constexpr int WS_MAX_QKV = 3 * 8192;
constexpr int WS_MAX_F = 65536;
constexpr int WS_MAX_GRID = 256;
constexpr int WS_MAX_HEADS = 128;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

int ws_alloc(Workspace& w) {
    size_t off = 0;
    auto take = [&](size_t bytes) {
        size_t o = off;
        off = align_up(off + bytes, 256);
        return o;
    };
    const size_t o_qkv = take(sizeof(uint2) * WS_MAX_QKV);
    const size_t o_mid = take(sizeof(float) * WS_MAX_F);
    const size_t o_hid0 = take(sizeof(uint2) * MAX_H);
    const size_t o_hid1 = take(sizeof(uint2) * MAX_H);
    const size_t o_part = take(sizeof(float) * WS_MAX_GRID * MAXL * (128 + 4));
    const size_t o_new = take(sizeof(float) * WS_MAX_HEADS * (128 + 4));
    const size_t o_av = take(sizeof(float) * WS_MAX_GRID);
    const size_t o_ai = take(sizeof(int) * WS_MAX_GRID);
    const size_t o_sync = take(sizeof(unsigned) * 4);
    const size_t o_stat = take(sizeof(int) * 4);
    char* b = nullptr;
    CF_CUDA(cudaMalloc(&b, off));
    CF_CUDA(cudaMemset(b, 0, off));
    w.base = b;
    w.qkv_ll = reinterpret_cast<uint2*>(b + o_qkv);
    w.mid_f32 = reinterpret_cast<float*>(b + o_mid);
    w.hid_ll[0] = reinterpret_cast<uint2*>(b + o_hid0);
    w.hid_ll[1] = reinterpret_cast<uint2*>(b + o_hid1);
    w.attn_part = reinterpret_cast<float*>(b + o_part);
    w.attn_new = reinterpret_cast<float*>(b + o_new);
    w.amax_val = reinterpret_cast<float*>(b + o_av);
    w.amax_idx = reinterpret_cast<int*>(b + o_ai);
    w.sync = reinterpret_cast<unsigned*>(b + o_sync);
    w.status = reinterpret_cast<int*>(b + o_stat);
    return CF_OK;
}

struct LaunchCfg {
    int cs = 0;
    int grid = 0;
    bool coop = true;
    bool ready = false;
};

const void* kernel_ptr(int D, int cs) {
    if (D == 80) {
        if (cs == 1) return reinterpret_cast<const void*>(&fused_decode_kernel<80, 1>);
        if (cs == 2) return reinterpret_cast<const void*>(&fused_decode_kernel<80, 2>);
        if (cs == 4) return reinterpret_cast<const void*>(&fused_decode_kernel<80, 4>);
    } else if (D == 128) {
        if (cs == 1) return reinterpret_cast<const void*>(&fused_decode_kernel<128, 1>);
        if (cs == 2) return reinterpret_cast<const void*>(&fused_decode_kernel<128, 2>);
        if (cs == 4) return reinterpret_cast<const void*>(&fused_decode_kernel<128, 4>);
    }
    return nullptr;
}

// several parameter blocks as one launch (head_dim 128 only: the Llama blocks)
const void* multi_kernel_ptr(int D, int cs) {
    if (D == 128) {
        if (cs == 1) return reinterpret_cast<const void*>(&fused_decode_multi_kernel<128, 1>);
        if (cs == 2) return reinterpret_cast<const void*>(&fused_decode_multi_kernel<128, 2>);
        if (cs == 4) return reinterpret_cast<const void*>(&fused_decode_multi_kernel<128, 4>);
    }
    return nullptr;
}

struct DescKey {
    const void* p[14];
    int64_t kv_rows;
    int dims[6];
    bool operator<(const DescKey& o) const { return memcmp(this, &o, sizeof(DescKey)) < 0; }
};

struct GraphCtx {
    int model;
    LayerDesc host;
    LayerDesc* dev = nullptr;
    __half *out = nullptr, *k_new = nullptr, *v_new = nullptr;
    const int* seq_dev = nullptr;
    const float *cos_t = nullptr, *sin_t = nullptr;
    int table_stride = 0;
    bool dirty = true;
};

struct DeviceState {
    int dev = -1;
    int sm_count = 0;
    int smem_optin = 0;
    LaunchCfg cfg[2];  // [0]: head_dim 80, [1]: head_dim 128
    Workspace ws;
    std::map<DescKey, LayerDesc*> desc_cache;
    // batches of recorded launches (cf_batch_begin / cf_batch_end): parameter blocks on the device, what they hold,
    // two pinned staging slots with the events of their last copies, the grid barrier's two words
    Params* multi_dev = nullptr;
    size_t multi_cap = 0;
    std::vector<Params> multi_last;
    Params* multi_pin[2] = {nullptr, nullptr};
    cudaEvent_t multi_ev[2] = {nullptr, nullptr};
    int multi_slot = 0;
    unsigned* multi_bar = nullptr;
    bool multi_attr[3] = {false, false, false};
    std::map<std::pair<int, int64_t>, GraphCtx> contexts;
    unsigned long long* trace = nullptr;  // diagnostics: timeline buffer applied to every launch
    size_t trace_slots = 0;
};

std::mutex g_mu;
std::unordered_map<int, DeviceState*> g_devices;

int env_int(const char* name, int dflt) {
    const char* v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

std::mutex g_cfg_mu;  // launch geometry is chosen once per (device, head_dim); serialise the choosing

int pick_cfg(DeviceState& ds, int D) {
    std::lock_guard<std::mutex> lk(g_cfg_mu);
    LaunchCfg& c = ds.cfg[D == 128];
    if (c.ready) return CF_OK;
    const int forced = env_int("CFB200_CLUSTER", 0);
    const int order[3] = {2, 4, 1};
    int best_cs = 0, best_cov = -1;
    for (int k = 0; k < 3; ++k) {
        const int cs = order[k];
        if (forced && cs != forced) continue;
        const void* fn = kernel_ptr(D, cs);
        CF_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, ds.smem_optin));
        int cov = 0;
        if (cs == 1) {
            int nb = 0;
            CF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, fn, NTHREADS, ds.smem_optin));
            cov = nb > 0 ? ds.sm_count : 0;
        } else {
            cudaLaunchConfig_t lc = {};
            lc.gridDim = dim3((ds.sm_count / cs) * cs);
            lc.blockDim = dim3(NTHREADS);
            lc.dynamicSmemBytes = ds.smem_optin;
            cudaLaunchAttribute at[1];
            at[0].id = cudaLaunchAttributeClusterDimension;
            at[0].val.clusterDim.x = cs;
            at[0].val.clusterDim.y = 1;
            at[0].val.clusterDim.z = 1;
            lc.attrs = at;
            lc.numAttrs = 1;
            int ncl = 0;
            CF_CUDA(cudaOccupancyMaxActiveClusters(&ncl, fn, &lc));
            cov = ncl * cs;
            if (cov > (ds.sm_count / cs) * cs) cov = (ds.sm_count / cs) * cs;
        }
        if (cov > best_cov) {
            best_cov = cov;
            best_cs = cs;
        }
    }
    if (best_cov <= 0) return fail(CF_ERR_CUDA, "no launch geometry fits on this device (head_dim %d)", D);
    const int cap = env_int("CFB200_GRID", 0);
    if (cap > 0 && cap < best_cov) best_cov = (cap / best_cs) * best_cs;
    c.cs = best_cs;
    c.grid = best_cov;
    c.coop = env_int("CFB200_COOPERATIVE", 1) != 0;
    c.ready = true;
    return CF_OK;
}

int get_device(DeviceState** out) {
    int dev = -1;
    CF_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_devices.find(dev);
    if (it != g_devices.end()) {
        *out = it->second;
        return CF_OK;
    }
    cudaDeviceProp prop;
    CF_CUDA(cudaGetDeviceProperties(&prop, dev));
    if (prop.major != 10)
        return fail(CF_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev, prop.major,
                    prop.minor);
    {
        const int ns = env_int("CFB200_POLL_BACKOFF_NS", -1);
        if (ns >= 0) CF_CUDA(cudaMemcpyToSymbol(c_poll_backoff_ns, &ns, sizeof(int)));
    }
    DeviceState* ds = new DeviceState();
    ds->dev = dev;
    ds->sm_count = prop.multiProcessorCount;
    int optin = 0;
    CF_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    ds->smem_optin = optin;
    int rc = ws_alloc(ds->ws);
    if (rc != CF_OK) {
        delete ds;
        return rc;
    }
    g_devices[dev] = ds;
    *out = ds;
    return CF_OK;
}

int check_dims(const CfDims& d) {
    if (d.head_dim != 80 && d.head_dim != 128) return fail(CF_ERR_UNSUPPORTED, "head_dim %d (80 or 128)", d.head_dim);
    if (d.hidden <= 0 || d.hidden % KCHUNK != 0 || d.hidden > MAX_H)
        return fail(CF_ERR_INVALID, "hidden %d must be a multiple of %d and at most %d", d.hidden, KCHUNK, MAX_H);
    if (d.heads <= 0 || d.heads > WS_MAX_HEADS || 3 * d.heads * d.head_dim > WS_MAX_QKV)
        return fail(CF_ERR_INVALID, "heads %d out of range", d.heads);
    if (d.ffn < 0 || d.ffn % GRAN != 0 || d.ffn > WS_MAX_F) return fail(CF_ERR_INVALID, "ffn %d out of range", d.ffn);
    if (d.rotary < 0 || d.rotary > d.head_dim || (d.rotary & 1)) return fail(CF_ERR_INVALID, "rotary %d", d.rotary);
    return CF_OK;
}

// ring depth and activation buffer for one launch
// cf_batch_begin .. cf_batch_end on this thread: launch() records the finished parameter block instead of launching
struct Recorded {
    Params p;
    size_t smem;
    int head_dim, cs, grid;
};
thread_local bool tl_recording = false;
thread_local std::vector<Recorded> tl_rec;
constexpr size_t MULTI_PARAMS_SLOT = (sizeof(Params) + 127) / 128 * 128;  // the blocks' copy in shared memory

int fit_smem(const DeviceState& ds, const CfDims& d, int cs, int p3_flags, int* nstage, int* xbuf_floats, int* aux_off) {
    const int KVW = d.heads * d.head_dim;
    const int kco = (p3_flags & F3_USE_O) ? ceil_div(KVW, KCHUNK) : 0;
    const int kc3 = kco + ((p3_flags & F3_USE_DOWN) ? ceil_div(d.ffn, KCHUNK) : 0);
    int xb = 2 * d.hidden;  // both LayerNorm outputs of a layer side by side
    if (ceil_div(kc3, cs) * KCHUNK > xb) xb = ceil_div(kc3, cs) * KCHUNK;
    // The auxiliary region (pre-staged queries + hand-over buffer of attention partials) must stay clear
    // of the LayerNorm outputs and of the MLP chunks a CTA stages at the start of P3, which are the
    // first (chunks it owns) - (attention chunks it owns) chunks of xbuf.
    int nmid_max = 0;
    for (int me = 0; me < cs; ++me) {
        const int my3 = kc3 > me ? ceil_div(kc3 - me, cs) : 0, nattn = kco > me ? ceil_div(kco - me, cs) : 0;
        if (my3 - nattn > nmid_max) nmid_max = my3 - nattn;
    }
    int aux = 2 * d.hidden;
    if (nmid_max * KCHUNK > aux) aux = nmid_max * KCHUNK;
    aux = (aux + 3) / 4 * 4;
    if (aux + aux_floats(d.head_dim) > xb) xb = aux + aux_floats(d.head_dim);
    *aux_off = aux;
    xb = (xb + 3) / 4 * 4;
    const long fixed = static_cast<long>(smem_bytes_for(0, xb));
    const long avail = ds.smem_optin - (tl_recording ? static_cast<long>(MULTI_PARAMS_SLOT) + 128 : 0);
    int ns = static_cast<int>((avail - fixed) / STAGE_BYTES);
    const int cap = env_int("CFB200_STAGES", 0);
    if (cap > 0 && ns > cap) ns = cap;
    if (ns > MAX_STAGES) ns = MAX_STAGES;
    if (ns < 2) return fail(CF_ERR_UNSUPPORTED, "shared memory too small: %d bytes for %d activation floats", ds.smem_optin, xb);
    *nstage = ns;
    *xbuf_floats = xb;
    return CF_OK;
}

int launch(DeviceState& ds, const CfDims& d, Params& p, cudaStream_t st) {
    int rc = pick_cfg(ds, d.head_dim);
    if (rc != CF_OK) return rc;
    LaunchCfg& c = ds.cfg[d.head_dim == 128];
    if (d.heads > c.grid) return fail(CF_ERR_UNSUPPORTED, "more heads (%d) than CTAs (%d)", d.heads, c.grid);
    if (ceil_div(d.hidden / GRAN, c.grid / c.cs) * GRAN > MAX_P3_ROWS)
        return fail(CF_ERR_UNSUPPORTED, "hidden %d too wide for %d clusters", d.hidden, c.grid / c.cs);
    {
        const int kco = ceil_div(d.heads * d.head_dim, KCHUNK);
        const int hpc = heads_per_chunk(d.head_dim);
        const int pstr = ceil_div(c.grid, d.heads) + 2;
        if (pstr > MAX_PARTS || ceil_div(kco, c.cs) * hpc * pstr > WTS_SLOTS)
            return fail(CF_ERR_UNSUPPORTED, "attention merge table too small for %d heads on %d CTAs", d.heads, c.grid);
    }
    {
        // joint QKV + MLP-up row split: usable when the derived up ranges are monotone
        const int ngq = (p.arch_flags & AF_NO_QKV) ? 0 : 3 * d.heads * d.head_dim / GRAN;
        const int ng1 = ngq + (p.F_up ? p.F_up : d.ffn) / GRAN;
        bool ok = true;
        int prev = 0;
        for (int i = 1; i <= c.grid && ok; ++i) {
            const int u = part_begin(i, ng1, c.grid) - part_begin(i, ngq, c.grid);
            ok = u >= prev;
            prev = u;
        }
        // Measured on B200: grouping the CTAs by matrix beats giving every CTA both matrices for
        // Pythia-6.9B on 1, 4 and 8 GPUs (0.4 - 6 %), ties on 2 GPUs, loses 1.5 % for Pythia-2.8B.
        p.p1_joint = 2;  // grouped; 1 / 0 (every CTA both matrices) stay selectable for experiments
        (void)ok;
        // Grouped split: attention needs only q/k/v, which the QKV group produces.  Give that group one
        // granule per CTA less than the average, so that q/k/v exist by the time the MLP-up group reaches
        // attention and nobody polls for long.
        {
            // ... but never more than 10 % less, which matters for small shards
            const double avg = static_cast<double>(ng1) / c.grid;
            const double per_q = (avg - 1.0 > 0.9 * avg) ? avg - 1.0 : 0.9 * avg;
            int gq = (ngq > 0 && ng1 > ngq) ? static_cast<int>(ngq / per_q + 0.999) : c.grid;
            if (gq < 1) gq = 1;
            const int forced = env_int("CFB200_GQ", 0);
            if (forced > 0) gq = forced;
            p.gq = gq;
        }
        const int mode = env_int("CFB200_P1_MODE", -1);
        if (mode == 0 || mode == 2 || mode == 3 || (mode == 1 && ok)) p.p1_joint = mode;
    }
    rc = fit_smem(ds, d, c.cs, p.p3_flags, &p.nstage, &p.xbuf_floats, &p.aux_off);
    if (rc != CF_OK) return rc;
    const size_t smem = smem_bytes_for(p.nstage, p.xbuf_floats);
    const void* fn = kernel_ptr(d.head_dim, c.cs);
    p.qkv_any_epoch = (p.phase_mask & PH_P1) ? 0 : 1;
    p.part_any_epoch = (p.phase_mask & PH_P2) ? 0 : 1;
    // CFB200_PDL=1: per-layer launches (never the whole-token decoder, whose predecessor writes the token and the
    // sequence length) are chained by programmatic dependent launch
    p.pdl = (env_int("CFB200_PDL", 0) != 0 && !(p.phase_mask & PH_P4) && p.tp_size <= 1) ? 1 : 0;
    p.merge_seg_max = env_int("CFB200_MERGE_SEG", 0);
    p.trace = nullptr;
    if (tl_recording) {
        if ((p.phase_mask & PH_P4) || p.tp_size > 1)
            return fail(CF_ERR_UNSUPPORTED, "whole-token and tensor-parallel launches cannot be part of a batch");
        if (!multi_kernel_ptr(d.head_dim, c.cs)) return fail(CF_ERR_UNSUPPORTED, "batches need head_dim 128");
        if (tl_rec.size() >= 4096) return fail(CF_ERR_UNSUPPORTED, "more than 4096 launches in one batch");
        p.pdl = 0;
        Recorded r;
        r.p = p;
        r.smem = smem;
        r.head_dim = d.head_dim;
        r.cs = c.cs;
        r.grid = c.grid;
        tl_rec.push_back(r);
        return CF_OK;
    }
    if (ds.trace && static_cast<size_t>(c.grid) * (p.n_layers + 1) * TRACE_EVENTS <= ds.trace_slots) p.trace = ds.trace;
    for (int attempt = 0; attempt < 2; ++attempt) {
        cudaLaunchConfig_t lc = {};
        lc.gridDim = dim3(c.grid);
        lc.blockDim = dim3(NTHREADS);
        lc.dynamicSmemBytes = smem;
        lc.stream = st;
        cudaLaunchAttribute at[3];
        int na = 0;
        if (c.cs > 1) {
            at[na].id = cudaLaunchAttributeClusterDimension;
            at[na].val.clusterDim.x = c.cs;
            at[na].val.clusterDim.y = 1;
            at[na].val.clusterDim.z = 1;
            ++na;
        }
        if (p.pdl) {
            // may start while the preceding kernel drains (never together with a cooperative launch: the
            // grid is sized from the occupancy query, so it is co-resident once that kernel has left)
            at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            at[na].val.programmaticStreamSerializationAllowed = 1;
            ++na;
        } else if (c.coop) {
            at[na].id = cudaLaunchAttributeCooperative;
            at[na].val.cooperative = 1;
            ++na;
        }
        lc.attrs = at;
        lc.numAttrs = na;
        void* args[1] = {&p};
        cudaError_t e = cudaLaunchKernelExC(&lc, fn, args);
        if (e == cudaSuccess) return CF_OK;
        if (c.coop && attempt == 0) {
            // cooperative + cluster launch refused: the grid is sized from the
            // occupancy query, so co-residency still holds without the attribute
            (void)cudaGetLastError();
            c.coop = false;
            continue;
        }
        return fail(CF_ERR_CUDA, "kernel launch failed: %s (grid %d, cluster %d, smem %zu)", cudaGetErrorString(e),
                    c.grid, c.cs, smem);
    }
    return CF_OK;
}

void base_params(Params& p, const CfDims& d, const Workspace& ws) {
    memset(&p, 0, sizeof(p));
    p.H = d.hidden;
    p.NH = d.heads;
    p.R = d.rotary;
    p.F = d.ffn;
    p.qkv_ll = ws.qkv_ll;
    p.epoch_base = ws.sync + 2;
    p.hid_ll[0] = ws.hid_ll[0];
    p.hid_ll[1] = ws.hid_ll[1];
    p.mid_f32 = ws.mid_f32;
    p.attn_part = ws.attn_part;
    p.attn_new = ws.attn_new;
    p.sync = ws.sync;
    p.status = ws.status;
    p.amax_val = ws.amax_val;
    p.amax_idx = ws.amax_idx;
}

// Tensor map of a key or value cache [kv_rows][heads * head_dim]: boxes of one head x KV_TILE rows.
int encode_kv(CUtensorMap* tm, const CfDims& d, void* cache, int64_t kv_rows) {
    const int KVW = d.heads * d.head_dim;
    // a head's slice of a cache row is head_dim * 2 bytes: promote L2 fetches to 256 B only when
    // that is a whole number of 256-byte lines (head_dim 128), otherwise fetch exact sectors
    const CUtensorMapL2promotion kvp =
        (d.head_dim * 2) % 256 == 0 ? CU_TENSOR_MAP_L2_PROMOTION_L2_256B : CU_TENSOR_MAP_L2_PROMOTION_NONE;
    return encode_2d(tm, cache, KVW, kv_rows, KVW, d.head_dim, KV_TILE, kvp);
}

// Build the six tensor maps + pointers of one layer.  Null matrices are skipped.
int build_layer_desc(LayerDesc& L, const CfDims& d, const CfLayerWeights& w, void* k_cache, void* v_cache,
                     int64_t kv_rows, int up_rows = 0) {
    memset(&L, 0, sizeof(L));
    const int KVW = d.heads * d.head_dim;
    int rc;
    if (w.qkv_weight && (rc = encode_weight(&L.tm_qkv, w.qkv_weight, d.hidden, 3 * KVW))) return rc;
    if (w.mlp_up_weight && (rc = encode_weight(&L.tm_up, w.mlp_up_weight, d.hidden, up_rows ? up_rows : d.ffn))) return rc;
    if (w.o_weight && (rc = encode_weight(&L.tm_o, w.o_weight, KVW, d.hidden))) return rc;
    if (w.mlp_down_weight && (rc = encode_weight(&L.tm_down, w.mlp_down_weight, d.ffn, d.hidden))) return rc;
    if (k_cache && (rc = encode_kv(&L.tm_k, d, k_cache, kv_rows))) return rc;
    if (v_cache && (rc = encode_kv(&L.tm_v, d, v_cache, kv_rows))) return rc;
    L.ln_w = static_cast<const __half*>(w.ln_weight);
    L.ln_b = static_cast<const __half*>(w.ln_bias);
    L.pln_w = static_cast<const __half*>(w.post_ln_weight);
    L.pln_b = static_cast<const __half*>(w.post_ln_bias);
    L.b_qkv = static_cast<const __half*>(w.qkv_bias);
    L.b_up = static_cast<const __half*>(w.mlp_up_bias);
    L.b_o = static_cast<const __half*>(w.o_bias);
    L.b_down = static_cast<const __half*>(w.mlp_down_bias);
    L.k_cache = static_cast<__half*>(k_cache);
    L.v_cache = static_cast<__half*>(v_cache);
    L.kv_rows = static_cast<int>(kv_rows);
    return CF_OK;
}

// device-resident descriptor for an eager call; built once per distinct tensor set
int cached_desc(DeviceState& ds, const CfDims& d, const CfLayerWeights& w, void* k_cache, void* v_cache,
                int64_t kv_rows, cudaStream_t st, LayerDesc** out, int up_rows = 0) {
    DescKey key;
    memset(&key, 0, sizeof(key));
    const void* ptrs[14] = {w.qkv_weight, w.qkv_bias, w.o_weight, w.o_bias, w.ln_weight, w.ln_bias, w.post_ln_weight,
                            w.post_ln_bias, w.mlp_up_weight, w.mlp_up_bias, w.mlp_down_weight, w.mlp_down_bias,
                            k_cache, v_cache};
    memcpy(key.p, ptrs, sizeof(ptrs));
    key.kv_rows = kv_rows;
    key.dims[0] = d.hidden; key.dims[1] = d.heads; key.dims[2] = d.head_dim; key.dims[3] = d.ffn; key.dims[4] = d.rotary;
    key.dims[5] = up_rows;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = ds.desc_cache.find(key);
    if (it != ds.desc_cache.end()) {
        *out = it->second;
        return CF_OK;
    }
    {
        int rc = refuse_upload_in_capture(st, "layer call");
        if (rc != CF_OK) return rc;
    }
    if (ds.desc_cache.size() >= 1024) {  // callers that churn tensors: start over
        // entries may still be referenced by launches in flight
        CF_CUDA(cudaDeviceSynchronize());
        for (auto& kv : ds.desc_cache) cudaFree(kv.second);
        ds.desc_cache.clear();
    }
    LayerDesc host;
    int rc = build_layer_desc(host, d, w, k_cache, v_cache, kv_rows, up_rows);
    if (rc != CF_OK) return rc;
    LayerDesc* dev = nullptr;
    CF_CUDA(cudaMalloc(&dev, sizeof(LayerDesc)));
    cudaError_t e = cudaMemcpyAsync(dev, &host, sizeof(LayerDesc), cudaMemcpyHostToDevice, st);
    if (e != cudaSuccess) {
        cudaFree(dev);
        return fail(CF_ERR_CUDA, "descriptor upload failed: %s", cudaGetErrorString(e));
    }
    ds.desc_cache[key] = dev;
    *out = dev;
    return CF_OK;
}

int model_dims(int model, CfDims* d) {
    if (model != CF_PYTHIA_2B8 && model != CF_PYTHIA_6B9) return fail(CF_ERR_INVALID, "unknown model id %d", model);
    *d = kDims[model];
    return CF_OK;
}

int check_layer_args(const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, bool need_down, bool need_out) {
    if (!w || !io) return fail(CF_ERR_INVALID, "null argument struct");
    if (!w->qkv_weight || !w->qkv_bias || !w->o_weight || !w->o_bias || !w->ln_weight || !w->ln_bias ||
        !w->post_ln_weight || !w->post_ln_bias || !w->mlp_up_weight || !w->mlp_up_bias)
        return fail(CF_ERR_INVALID, "null weight pointer");
    if (need_down && (!w->mlp_down_weight || !w->mlp_down_bias)) return fail(CF_ERR_INVALID, "null mlp_down pointer");
    if (!io->input || !io->k_cache || !io->v_cache || !io->cos || !io->sin) return fail(CF_ERR_INVALID, "null io pointer");
    if (need_out && !io->output) return fail(CF_ERR_INVALID, "null output pointer");
    if (io->kv_rows <= 0 || io->kv_rows > 0x7fffffff) return fail(CF_ERR_INVALID, "kv_rows %lld", (long long)io->kv_rows);
    if (seq_len < 0 || seq_len >= io->kv_rows)
        return fail(CF_ERR_INVALID, "current_seq_len %lld outside [0, %lld): the cache needs a free row for the new token",
                    (long long)seq_len, (long long)io->kv_rows);
    return CF_OK;
}

constexpr int F3_FULL = F3_USE_O | F3_USE_DOWN | F3_ADD_X | F3_ADD_BO | F3_ADD_BDOWN;

int run_layer(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, void* stream, bool split) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if ((rc = check_layer_args(w, io, seq_len, true, true))) return rc;
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LayerDesc* desc;
    if ((rc = cached_desc(*ds, d, *w, io->k_cache, io->v_cache, io->kv_rows, st, &desc))) return rc;
    Params p;
    base_params(p, d, ds->ws);
    p.layers = desc;
    p.n_layers = 1;
    p.p3_flags = F3_FULL;
    p.x_in = static_cast<const __half*>(io->input);
    p.out = static_cast<__half*>(io->output);
    p.k_new = static_cast<__half*>(io->k_new);
    p.v_new = static_cast<__half*>(io->v_new);
    p.cos = io->cos;
    p.sin = io->sin;
    p.seq_host = static_cast<int>(seq_len);
    if (!split) {
        p.phase_mask = PH_P1 | PH_P2 | PH_P3;
        return launch(*ds, d, p, st);
    }
    p.phase_mask = PH_P1 | PH_P2;
    if ((rc = launch(*ds, d, p, st))) return rc;
    p.phase_mask = PH_P3;
    return launch(*ds, d, p, st);
}

// ---- small helper kernels of the tensor-parallel path
__global__ void embed_gather_kernel(const __half* embed, const int* token, __half* dst, int H) {
    const size_t row = static_cast<size_t>(*token) * H;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x) dst[i] = embed[row + i];
}
__global__ void tp_finish_kernel(const __half* x, const __half* partial, const __half* b_o, const __half* b_down,
                                 __half* out, int H) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < H; i += gridDim.x * blockDim.x)
        out[i] = __float2half_rn(__half2float(x[i]) + __half2float(partial[i]) + __half2float(b_o[i]) +
                                 __half2float(b_down[i]));
}
__global__ void select_token_kernel(const float* vals, const int* idxs, int n, int* token, int* seq) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        float b = vals[0];
        int bi = idxs[0];
        for (int i = 1; i < n; ++i)
            if (vals[i] > b || (vals[i] == b && idxs[i] < bi)) {
                b = vals[i];
                bi = idxs[i];
            }
        *token = bi;
        *seq += 1;
    }
}

struct Decoder {
    CfDecoderConfig cfg;
    int dev = -1;
    std::vector<LayerDesc> layers_h;
    std::vector<bool> layer_set;
    LayerDesc* layers_d = nullptr;
    TailDesc tail_h;
    TailDesc* tail_d = nullptr;
    CfHeadWeights head;
    bool head_set = false, finalized = false;
    Workspace ws;
    int *token_d = nullptr, *seq_d = nullptr;
    float* logits_d = nullptr;
    __half *hidden_d = nullptr, *hid0 = nullptr, *hid1 = nullptr, *partial_d = nullptr;
    // fused tensor-parallel exchange (peer memory over NVLink)
    unsigned char* tp_local = nullptr;          // this rank's exchange buffer (cudaMalloc, exported by IPC)
    unsigned char* tp_peer[MAX_TP] = {nullptr};  // every rank's buffer as mapped here ([tp_rank] == tp_local)
    unsigned* tp_count = nullptr;
    bool tp_connected = false;
    bool tp_ipc = false;  // peers were opened through CUDA IPC (and must be closed)
};

std::unordered_map<int64_t, Decoder*> g_decoders;
int64_t g_next_handle = 1;

int find_decoder(int64_t h, Decoder** out) {
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = g_decoders.find(h);
    if (it == g_decoders.end()) return fail(CF_ERR_INVALID, "unknown decoder handle %lld", (long long)h);
    *out = it->second;
    return CF_OK;
}

void decoder_params(Decoder& dc, Params& p) {
    base_params(p, dc.cfg.dims, dc.ws);
    p.cos = dc.cfg.cos_table;
    p.sin = dc.cfg.sin_table;
    p.rope_stride = dc.cfg.dims.rotary;
    p.seq_ptr = dc.seq_d;
    if (dc.cfg.flags & CF_DECODER_GELU_ERF) p.arch_flags |= AF_GELU_ERF;
}

// ---------------------------------------------------------------------------
// Scratch for cf_pythia_decoder_layer_noalloc: everything the fused layer kernel
// needs beyond its inputs and outputs, in one statically allocated device array.
// Sized for the two built-in models on a grid of at most NOALLOC_MAX_GRID CTAs.
// Every GPU that loads this library holds these bytes until the process exits.
constexpr int NOALLOC_MAX_GRID = 160;
constexpr int NOALLOC_MAX_HEADS = 32;
constexpr int NOALLOC_MAX_KVW = 4096;   // heads * head_dim
constexpr int NOALLOC_MAX_FFN = 16384;
constexpr size_t NA_OFF_QKV = 0;
constexpr size_t NA_OFF_MID = NA_OFF_QKV + sizeof(uint2) * 3 * NOALLOC_MAX_KVW;
constexpr size_t NA_OFF_PART = NA_OFF_MID + sizeof(float) * NOALLOC_MAX_FFN;
constexpr size_t NA_OFF_NEW = NA_OFF_PART + sizeof(float) * NOALLOC_MAX_GRID * MAXL * (128 + 4);
constexpr size_t NA_OFF_AMAXV = NA_OFF_NEW + sizeof(float) * NOALLOC_MAX_HEADS * (128 + 4);
constexpr size_t NA_OFF_AMAXI = NA_OFF_AMAXV + sizeof(float) * NOALLOC_MAX_GRID;
constexpr size_t NA_OFF_SYNC = NA_OFF_AMAXI + sizeof(int) * NOALLOC_MAX_GRID;   // 4 barrier words + 4 status words
constexpr size_t NA_OFF_DESC = (NA_OFF_SYNC + 32 + 255) / 256 * 256;            // one LayerDesc (tensor maps)
constexpr size_t NOALLOC_SCRATCH_BYTES = NA_OFF_DESC + sizeof(LayerDesc);
static_assert(NOALLOC_SCRATCH_BYTES <= 576 * 1024, "the static scratch is meant to stay modest");
static_assert(NA_OFF_MID % 256 == 0 && NA_OFF_PART % 256 == 0 && NA_OFF_NEW % 128 == 0 && NA_OFF_SYNC % 16 == 0,
              "sub-buffers must keep the alignment the kernel's vector loads and tensor maps need");

static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoAllocDevice {
    bool ready = false;
    unsigned char* scratch = nullptr;  // DEVICE address of g_noalloc_scratch on this GPU
    DeviceState ds;                    // launch geometry only; its workspace points into the scratch
    DescKey last_key;                  // what the descriptor slot currently holds
    bool have_key = false;
};
NoAllocDevice g_noalloc[NOALLOC_MAX_DEVICES];
std::mutex g_noalloc_mu;

// Once per device, with that device current.  In host code the array's name is only
// a stand-in, not a device address: the address has to be asked for.
int noalloc_setup(NoAllocDevice** out) {
    int dev = -1;
    CF_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= NOALLOC_MAX_DEVICES) return fail(CF_ERR_UNSUPPORTED, "device index %d", dev);
    NoAllocDevice& nd = g_noalloc[dev];
    if (!nd.ready) {
        cudaDeviceProp prop;
        CF_CUDA(cudaGetDeviceProperties(&prop, dev));
        if (prop.major != 10)
            return fail(CF_ERR_UNSUPPORTED, "device %d is sm_%d%d; this library is built for sm_100a only", dev,
                        prop.major, prop.minor);
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return fail(CF_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        nd.scratch = static_cast<unsigned char*>(ptr);
        nd.ds.dev = dev;
        nd.ds.sm_count = prop.multiProcessorCount;
        int optin = 0;
        CF_CUDA(cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
        nd.ds.smem_optin = optin;
        Workspace& w = nd.ds.ws;
        w.base = nd.scratch;
        w.qkv_ll = reinterpret_cast<uint2*>(nd.scratch + NA_OFF_QKV);
        w.mid_f32 = reinterpret_cast<float*>(nd.scratch + NA_OFF_MID);
        w.attn_part = reinterpret_cast<float*>(nd.scratch + NA_OFF_PART);
        w.attn_new = reinterpret_cast<float*>(nd.scratch + NA_OFF_NEW);
        w.amax_val = reinterpret_cast<float*>(nd.scratch + NA_OFF_AMAXV);
        w.amax_idx = reinterpret_cast<int*>(nd.scratch + NA_OFF_AMAXI);
        w.sync = reinterpret_cast<unsigned*>(nd.scratch + NA_OFF_SYNC);
        w.status = reinterpret_cast<int*>(nd.scratch + NA_OFF_SYNC + 16);
        nd.ready = true;
    }
    *out = &nd;
    return CF_OK;
}

}  // namespace

// ---- helpers shared with the other translation units (host_common.h)
CfEncodeTiledFn cf_host_encode_fn() { return get_encode(); }
int cf_host_fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    g_err = buf;
    return code;
}
int cf_host_refuse_in_capture(cudaStream_t st, const char* what) { return refuse_upload_in_capture(st, what); }

// =============================================================================
extern "C" {

const char* cf_last_error(void) { return g_err.c_str(); }

int cf_model_dims(int model, CfDims* out) {
    if (!out) return fail(CF_ERR_INVALID, "null out");
    return model_dims(model, out);
}

int cf_launch_info(int model, int* sm_count, int* grid, int* cluster, int* stages, int* smem_bytes) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    if ((rc = pick_cfg(*ds, d.head_dim))) return rc;
    const LaunchCfg& c = ds->cfg[d.head_dim == 128];
    int ns = 0, xb = 0, aux = 0;
    if ((rc = fit_smem(*ds, d, c.cs, F3_FULL, &ns, &xb, &aux))) return rc;
    if (sm_count) *sm_count = ds->sm_count;
    if (grid) *grid = c.grid;
    if (cluster) *cluster = c.cs;
    if (stages) *stages = ns;
    if (smem_bytes) *smem_bytes = static_cast<int>(smem_bytes_for(ns, xb));
    return CF_OK;
}

int cf_get_status(int* status) {
    if (!status) return fail(CF_ERR_INVALID, "null status");
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    CF_CUDA(cudaDeviceSynchronize());
    int worst = 0;
    auto probe = [&](Workspace& ws) -> int {
        int s = 0;
        CF_CUDA(cudaMemcpy(&s, ws.status, sizeof(int), cudaMemcpyDeviceToHost));
        if (s != 0) {
            worst = s;
            CF_CUDA(cudaMemset(ws.status, 0, sizeof(int)));
            CF_CUDA(cudaMemset(ws.sync, 0, 2 * sizeof(unsigned)));  // barrier words only: the launch count keeps counting
        }
        return CF_OK;
    };
    if ((rc = probe(ds->ws))) return rc;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        for (auto& kv : g_decoders)
            if (kv.second->dev == ds->dev && (rc = probe(kv.second->ws))) return rc;
    }
    {
        // the static scratch of the allocation-free entry point, once a call has set it up on this device
        std::lock_guard<std::mutex> lk(g_noalloc_mu);
        if (ds->dev >= 0 && ds->dev < NOALLOC_MAX_DEVICES && g_noalloc[ds->dev].ready &&
            (rc = probe(g_noalloc[ds->dev].ds.ws)))
            return rc;
    }
    {
        int s = 0;
        if ((rc = cf_host_lb_probe_status(ds->dev, &s))) return rc;
        if (s != 0) worst = s;
    }
    *status = worst;
    if (worst != 0)
        return fail(CF_ERR_DEVICE,
                    "device status %d (1-2 TMA ring, 3 grid barrier / flag wait, 4 cluster exchange, 5 bad seq_len, "
                    "6 drain, 7 tensor-parallel peer never answered)",
                    worst);
    return CF_OK;
}

int cf_pythia_decoder_layer(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, void* stream) {
    return run_layer(model, w, io, seq_len, stream, false);
}

int cf_pythia_decoder_layer_split(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len,
                                  void* stream) {
    return run_layer(model, w, io, seq_len, stream, true);
}

int cf_pythia_decoder_layer_noalloc(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len,
                                    void* stream) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if ((rc = check_layer_args(w, io, seq_len, true, true))) return rc;
    if (d.heads > NOALLOC_MAX_HEADS || d.heads * d.head_dim > NOALLOC_MAX_KVW || d.ffn > NOALLOC_MAX_FFN)
        return fail(CF_ERR_UNSUPPORTED,
                    "model too large for the static scratch (%zu bytes: at most %d heads, %d QKV columns, ffn %d)",
                    NOALLOC_SCRATCH_BYTES, NOALLOC_MAX_HEADS, NOALLOC_MAX_KVW, NOALLOC_MAX_FFN);
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocDevice* nd;
    if ((rc = noalloc_setup(&nd))) return rc;
    if ((rc = pick_cfg(nd->ds, d.head_dim))) return rc;
    if (nd->ds.cfg[d.head_dim == 128].grid > NOALLOC_MAX_GRID)
        return fail(CF_ERR_UNSUPPORTED, "this GPU runs %d CTAs; the static scratch holds partials for at most %d",
                    nd->ds.cfg[d.head_dim == 128].grid, NOALLOC_MAX_GRID);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // tensor maps + pointers of this call's tensors into the descriptor slot (a copy, not an allocation)
    DescKey key;
    memset(&key, 0, sizeof(key));
    const void* ptrs[14] = {w->qkv_weight, w->qkv_bias, w->o_weight, w->o_bias, w->ln_weight, w->ln_bias,
                            w->post_ln_weight, w->post_ln_bias, w->mlp_up_weight, w->mlp_up_bias, w->mlp_down_weight,
                            w->mlp_down_bias, io->k_cache, io->v_cache};
    memcpy(key.p, ptrs, sizeof(ptrs));
    key.kv_rows = io->kv_rows;
    key.dims[0] = d.hidden; key.dims[1] = d.heads; key.dims[2] = d.head_dim; key.dims[3] = d.ffn; key.dims[4] = d.rotary;
    LayerDesc* desc = reinterpret_cast<LayerDesc*>(nd->scratch + NA_OFF_DESC);
    const bool upload = !nd->have_key || memcmp(&key, &nd->last_key, sizeof(key)) != 0;
    if (upload && (rc = refuse_upload_in_capture(st, "noalloc layer call"))) return rc;
    // The array keeps whatever the last call left: the two barrier words must start at zero.  The
    // third sync word is the running base of the q/k/v epochs and keeps counting; the status word is
    // left alone so that a failure of an earlier launch stays readable until cf_get_status reports
    // (and clears) it.
    CF_CUDA(cudaMemsetAsync(nd->ds.ws.sync, 0, 8, st));
    if (upload) {
        LayerDesc host;
        if ((rc = build_layer_desc(host, d, *w, io->k_cache, io->v_cache, io->kv_rows))) return rc;
        CF_CUDA(cudaMemcpyAsync(desc, &host, sizeof(LayerDesc), cudaMemcpyHostToDevice, st));
        nd->last_key = key;
        nd->have_key = true;
    }
    Params p;
    base_params(p, d, nd->ds.ws);
    p.layers = desc;
    p.n_layers = 1;
    p.p3_flags = F3_FULL;
    p.phase_mask = PH_P1 | PH_P2 | PH_P3;
    p.x_in = static_cast<const __half*>(io->input);
    p.out = static_cast<__half*>(io->output);
    p.k_new = static_cast<__half*>(io->k_new);
    p.v_new = static_cast<__half*>(io->v_new);
    p.cos = io->cos;
    p.sin = io->sin;
    p.seq_host = static_cast<int>(seq_len);
    return launch(nd->ds, d, p, st);
}

int cf_llama_decoder_layer_sglang(const void* input, const void* residual, const void* weight_qkv,
                                  const void* weight_o, const void* k_cache, const void* v_cache, int64_t seq_len,
                                  const void* rms_input_weight, float eps, const float* cos, const float* sin,
                                  void* output, void* residual_out, void* k_new, void* v_new, void* stream) {
    const CfDims d = {4096, 32, 128, 128, 0, 0};  // include/5090/llama/config.h:1-4 of the reference
    if (!input || !weight_qkv || !weight_o || !k_cache || !v_cache || !rms_input_weight || !cos || !sin || !output ||
        !residual_out)
        return fail(CF_ERR_INVALID, "null pointer");
    if (residual && residual == residual_out) return fail(CF_ERR_INVALID, "residual_out must not alias residual");
    if (seq_len < 1 || seq_len > 0x7fffffff)
        return fail(CF_ERR_INVALID, "the caches must hold at least one row (got %lld)", (long long)seq_len);
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CfLayerWeights w;
    memset(&w, 0, sizeof(w));
    w.qkv_weight = weight_qkv;
    w.o_weight = weight_o;
    w.ln_weight = rms_input_weight;
    LayerDesc* desc;
    // the descriptor holds the weights only (one per layer, whatever the sequence length); the caches, which
    // this entry point takes with exactly seq_len rows, get their tensor maps in the kernel parameters
    if ((rc = cached_desc(*ds, d, w, nullptr, nullptr, 0, st, &desc))) return rc;
    Params p;
    base_params(p, d, ds->ws);
    if ((rc = encode_kv(&p.kv_maps[0], d, const_cast<void*>(k_cache), seq_len))) return rc;
    if ((rc = encode_kv(&p.kv_maps[1], d, const_cast<void*>(v_cache), seq_len))) return rc;
    p.kv_inline = 1;
    p.kv_rows_inline = static_cast<int>(seq_len);
    p.layers = desc;
    p.n_layers = 1;
    p.phase_mask = PH_P1 | PH_P2 | PH_P3;
    p.p3_flags = F3_USE_O;
    p.arch_flags = AF_RMS_ADD | AF_QKV_PLANAR | AF_NO_APPEND;
    p.norm_eps = eps;
    p.x_in = static_cast<const __half*>(input);
    p.residual_in = static_cast<const __half*>(residual);
    p.residual_out = static_cast<__half*>(residual_out);
    p.out = static_cast<__half*>(output);
    p.k_new = static_cast<__half*>(k_new);
    p.v_new = static_cast<__half*>(v_new);
    p.cos = cos;
    p.sin = sin;
    p.seq_host = static_cast<int>(seq_len);
    return launch(*ds, d, p, st);
}

int cf_batch_begin(void) {
    if (tl_recording) return fail(CF_ERR_INVALID, "cf_batch_begin: a batch is already open on this thread");
    tl_rec.clear();
    tl_recording = true;
    return CF_OK;
}

int cf_batch_abort(void) {
    tl_recording = false;
    tl_rec.clear();
    return CF_OK;
}

int cf_batch_end(void* stream) {
    if (!tl_recording) return fail(CF_ERR_INVALID, "cf_batch_end without cf_batch_begin");
    tl_recording = false;
    std::vector<Recorded> rec;
    rec.swap(tl_rec);
    if (rec.empty()) return CF_OK;
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int n = static_cast<int>(rec.size());
    size_t smem = 0;
    for (const Recorded& r : rec) {
        if (r.head_dim != rec[0].head_dim || r.cs != rec[0].cs || r.grid != rec[0].grid)
            return fail(CF_ERR_UNSUPPORTED, "the launches of a batch must share head_dim and launch geometry");
        if (r.smem > smem) smem = r.smem;
    }
    const size_t params_off = align_up(smem, 128);
    const size_t dyn = params_off + MULTI_PARAMS_SLOT;
    if (dyn > static_cast<size_t>(ds->smem_optin))
        return fail(CF_ERR_UNSUPPORTED, "batch needs %zu bytes of shared memory (%d available)", dyn, ds->smem_optin);
    const void* fn = multi_kernel_ptr(rec[0].head_dim, rec[0].cs);
    std::lock_guard<std::mutex> lk(g_mu);
    const int ai = rec[0].cs == 1 ? 0 : (rec[0].cs == 2 ? 1 : 2);
    if (!ds->multi_attr[ai]) {
        CF_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, ds->smem_optin));
        ds->multi_attr[ai] = true;
    }
    // the blocks on the device: uploaded only when they differ from what is there (a captured graph replays an
    // identical batch without any copy; a batch that differs cannot be captured)
    bool same = ds->multi_last.size() == rec.size();
    for (int i = 0; same && i < n; ++i) same = memcmp(&ds->multi_last[i], &rec[i].p, sizeof(Params)) == 0;
    if (!same) {
        if ((rc = refuse_upload_in_capture(st, "a batch whose parameters changed"))) return rc;
        if (static_cast<size_t>(n) > ds->multi_cap) {
            const size_t cap = align_up(static_cast<size_t>(n), 64);
            CF_CUDA(cudaDeviceSynchronize());  // earlier batches may still read the old buffers
            if (ds->multi_dev) cudaFree(ds->multi_dev);
            for (int k = 0; k < 2; ++k) {
                if (ds->multi_pin[k]) cudaFreeHost(ds->multi_pin[k]);
                ds->multi_pin[k] = nullptr;
                if (!ds->multi_ev[k]) CF_CUDA(cudaEventCreateWithFlags(&ds->multi_ev[k], cudaEventDisableTiming));
            }
            ds->multi_dev = nullptr;
            ds->multi_cap = 0;
            CF_CUDA(cudaMalloc(&ds->multi_dev, cap * sizeof(Params)));
            for (int k = 0; k < 2; ++k) CF_CUDA(cudaMallocHost(&ds->multi_pin[k], cap * sizeof(Params)));
            ds->multi_cap = cap;
        }
        if (!ds->multi_bar) {
            CF_CUDA(cudaMalloc(&ds->multi_bar, 256));
            CF_CUDA(cudaMemset(ds->multi_bar, 0, 256));
        }
        const int slot = ds->multi_slot;
        ds->multi_slot ^= 1;
        CF_CUDA(cudaEventSynchronize(ds->multi_ev[slot]));  // the copy that last read this staging slot is over
        for (int i = 0; i < n; ++i) ds->multi_pin[slot][i] = rec[i].p;
        CF_CUDA(cudaMemcpyAsync(ds->multi_dev, ds->multi_pin[slot], static_cast<size_t>(n) * sizeof(Params),
                                cudaMemcpyHostToDevice, st));
        CF_CUDA(cudaEventRecord(ds->multi_ev[slot], st));
        ds->multi_last.resize(n);
        for (int i = 0; i < n; ++i) ds->multi_last[i] = rec[i].p;
    }
    MultiArgs ma;
    ma.blocks = ds->multi_dev;
    ma.n_blocks = n;
    ma.params_off = static_cast<int>(params_off);
    ma.bar = ds->multi_bar;
    ma.status = ds->ws.status;
    cudaLaunchConfig_t lc = {};
    lc.gridDim = dim3(rec[0].grid);
    lc.blockDim = dim3(NTHREADS);
    lc.dynamicSmemBytes = dyn;
    lc.stream = st;
    cudaLaunchAttribute at[2];
    int na = 0;
    if (rec[0].cs > 1) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = rec[0].cs;
        at[na].val.clusterDim.y = 1;
        at[na].val.clusterDim.z = 1;
        ++na;
    }
    LaunchCfg& c = ds->cfg[rec[0].head_dim == 128];
    if (c.coop) {
        at[na].id = cudaLaunchAttributeCooperative;
        at[na].val.cooperative = 1;
        ++na;
    }
    lc.attrs = at;
    lc.numAttrs = na;
    void* args[1] = {&ma};
    cudaError_t e = cudaLaunchKernelExC(&lc, fn, args);
    if (e != cudaSuccess && c.coop) {
        (void)cudaGetLastError();
        lc.numAttrs = na - 1;  // without the cooperative attribute: the grid is sized from the occupancy query
        e = cudaLaunchKernelExC(&lc, fn, args);
    }
    if (e != cudaSuccess)
        return fail(CF_ERR_CUDA, "batch launch failed: %s (%d blocks, grid %d, smem %zu)", cudaGetErrorString(e), n, rec[0].grid, dyn);
    return CF_OK;
}

int cf_llama_mlp_sglang(const void* input, const void* residual, const void* gate_up_weight, const void* down_weight,
                        const void* rms_weight, float eps, int64_t ffn, void* output, void* residual_out, void* stream) {
    if (!input || !gate_up_weight || !down_weight || !rms_weight || !output || !residual_out)
        return fail(CF_ERR_INVALID, "null pointer");
    if (residual && residual == residual_out) return fail(CF_ERR_INVALID, "residual_out must not alias residual");
    if (ffn <= 0 || (ffn % GRAN) != 0 || 2 * ffn > WS_MAX_F)
        return fail(CF_ERR_INVALID, "ffn %lld must be a positive multiple of %d and at most %d", (long long)ffn, GRAN, WS_MAX_F / 2);
    const CfDims d = {4096, 32, 128, 128, static_cast<int>(ffn), 0};  // hidden of include/5090/llama/config.h:1-4
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CfLayerWeights w;
    memset(&w, 0, sizeof(w));
    w.mlp_up_weight = gate_up_weight;
    w.mlp_down_weight = down_weight;
    w.ln_weight = rms_weight;
    LayerDesc* desc;
    if ((rc = cached_desc(*ds, d, w, nullptr, nullptr, 0, st, &desc, 2 * d.ffn))) return rc;
    Params p;
    base_params(p, d, ds->ws);
    p.layers = desc;
    p.n_layers = 1;
    p.phase_mask = PH_P1 | PH_P3;
    p.p3_flags = F3_USE_DOWN;
    p.arch_flags = AF_RMS_ADD | AF_NO_QKV | AF_SWIGLU;
    p.F_up = 2 * d.ffn;
    p.norm_eps = eps;
    p.x_in = static_cast<const __half*>(input);
    p.residual_in = static_cast<const __half*>(residual);
    p.residual_out = static_cast<__half*>(residual_out);
    p.out = static_cast<__half*>(output);
    p.seq_host = 0;
    return launch(*ds, d, p, st);
}

int cf_debug_run_phases(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, int phase_mask,
                        void* stream) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if ((rc = check_layer_args(w, io, seq_len, true, true))) return rc;
    if (phase_mask <= 0 || phase_mask > (PH_P1 | PH_P2 | PH_P3)) return fail(CF_ERR_INVALID, "phase_mask %d", phase_mask);
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    LayerDesc* desc;
    if ((rc = cached_desc(*ds, d, *w, io->k_cache, io->v_cache, io->kv_rows, st, &desc))) return rc;
    Params p;
    base_params(p, d, ds->ws);
    p.layers = desc;
    p.n_layers = 1;
    p.p3_flags = F3_FULL;
    p.phase_mask = phase_mask;
    p.x_in = static_cast<const __half*>(io->input);
    p.out = static_cast<__half*>(io->output);
    p.k_new = static_cast<__half*>(io->k_new);
    p.v_new = static_cast<__half*>(io->v_new);
    p.cos = io->cos;
    p.sin = io->sin;
    p.seq_host = static_cast<int>(seq_len);
    return launch(*ds, d, p, st);
}

int cf_debug_stream_rows(const void* matrix, int64_t rows, int64_t cols, const void* x, int touch_only,
                         void* scratch_desc, void* stream) {
    if (!matrix || !x || !scratch_desc) return fail(CF_ERR_INVALID, "null pointer");
    if (rows <= 0 || rows > 0x7fffffff || (rows % GRAN) != 0) return fail(CF_ERR_INVALID, "rows %lld", (long long)rows);
    if (cols <= 0 || cols > MAX_H || (cols % KCHUNK) != 0) return fail(CF_ERR_INVALID, "cols %lld", (long long)cols);
    if (reinterpret_cast<uintptr_t>(scratch_desc) & 127) return fail(CF_ERR_INVALID, "scratch_desc must be 128-byte aligned");
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if ((rc = refuse_upload_in_capture(st, "cf_debug_stream_rows"))) return rc;
    TailDesc host;
    memset(&host, 0, sizeof(host));
    if ((rc = encode_weight(&host.tm_head, matrix, static_cast<uint64_t>(cols), static_cast<uint64_t>(rows)))) return rc;
    // LayerNorm parameters of the tail: the activation vector itself serves (only the stream is timed)
    host.fln_w = static_cast<const __half*>(x);
    host.fln_b = static_cast<const __half*>(x);
    host.vocab = static_cast<int>(rows);
    CF_CUDA(cudaMemcpyAsync(scratch_desc, &host, sizeof(TailDesc), cudaMemcpyHostToDevice, st));
    CF_CUDA(cudaStreamSynchronize(st));  // `host` leaves scope
    const CfDims d = {static_cast<int>(cols), 32, 128, 0, 0, static_cast<int>(rows)};  // heads: launch-geometry checks only
    Params p;
    base_params(p, d, ds->ws);
    p.tail = static_cast<const TailDesc*>(scratch_desc);
    p.n_layers = 0;
    p.phase_mask = PH_P4;
    p.x_in = static_cast<const __half*>(x);
    p.touch_only = touch_only ? 1 : 0;
    return launch(*ds, d, p, st);
}

int cf_debug_set_trace(void* device_buffer, int64_t n_slots) {
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    ds->trace = static_cast<unsigned long long*>(device_buffer);
    ds->trace_slots = device_buffer ? static_cast<size_t>(n_slots) : 0;
    return CF_OK;
}

int cf_pythia_attention_only(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, void* stream) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if ((rc = check_layer_args(w, io, seq_len, false, false))) return rc;
    if (!io->attn_output || !io->mlp_intermediate) return fail(CF_ERR_INVALID, "null attn_output / mlp_intermediate");
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CfLayerWeights w2 = *w;
    w2.mlp_down_weight = nullptr;
    w2.mlp_down_bias = nullptr;
    LayerDesc* desc;
    if ((rc = cached_desc(*ds, d, w2, io->k_cache, io->v_cache, io->kv_rows, st, &desc))) return rc;
    Params p;
    base_params(p, d, ds->ws);
    p.layers = desc;
    p.n_layers = 1;
    p.phase_mask = PH_P1 | PH_P2 | PH_P3;
    p.p3_flags = F3_USE_O | F3_ADD_BO;
    p.x_in = static_cast<const __half*>(io->input);
    p.out = static_cast<__half*>(io->attn_output);
    p.mid_f16_out = static_cast<__half*>(io->mlp_intermediate);
    p.k_new = static_cast<__half*>(io->k_new);
    p.v_new = static_cast<__half*>(io->v_new);
    p.cos = io->cos;
    p.sin = io->sin;
    p.seq_host = static_cast<int>(seq_len);
    return launch(*ds, d, p, st);
}

int cf_pythia_mlp_only(int model, const void* input, const void* attn_output, const void* mlp_intermediate,
                       const void* mlp_down_weight, const void* mlp_down_bias, void* output, void* stream) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if (!input || !attn_output || !mlp_intermediate || !mlp_down_weight || !mlp_down_bias || !output)
        return fail(CF_ERR_INVALID, "null pointer");
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    CfLayerWeights w;
    memset(&w, 0, sizeof(w));
    w.mlp_down_weight = mlp_down_weight;
    w.mlp_down_bias = mlp_down_bias;
    LayerDesc* desc;
    if ((rc = cached_desc(*ds, d, w, nullptr, nullptr, 1, st, &desc))) return rc;
    Params p;
    base_params(p, d, ds->ws);
    p.layers = desc;
    p.n_layers = 1;
    p.phase_mask = PH_P3;
    p.p3_flags = F3_USE_DOWN | F3_ADD_X | F3_ADD_BDOWN | F3_MID_F16;
    p.x_in = static_cast<const __half*>(input);
    p.out = static_cast<__half*>(output);
    p.mid_f16_in = static_cast<const __half*>(mlp_intermediate);
    p.extra_add_f16 = static_cast<const __half*>(attn_output);
    p.cos = nullptr;
    p.sin = nullptr;
    p.seq_host = 0;
    return launch(*ds, d, p, st);
}

int cf_pythia_create_graph_context(int model, int64_t context_id, void* k_cache, void* v_cache,
                                   const void* weight_qkv, const void* weight_o, const void* mlp_up_weight,
                                   const void* mlp_down_weight, int64_t max_seq_len) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if (!k_cache || !v_cache || !weight_qkv || !weight_o || !mlp_up_weight || !mlp_down_weight)
        return fail(CF_ERR_INVALID, "null pointer");
    if (max_seq_len <= 0 || max_seq_len > 0x7fffffff) return fail(CF_ERR_INVALID, "max_seq_len %lld", (long long)max_seq_len);
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    GraphCtx ctx;
    ctx.model = model;
    CfLayerWeights w;
    memset(&w, 0, sizeof(w));
    w.qkv_weight = weight_qkv;
    w.o_weight = weight_o;
    w.mlp_up_weight = mlp_up_weight;
    w.mlp_down_weight = mlp_down_weight;
    if ((rc = build_layer_desc(ctx.host, d, w, k_cache, v_cache, max_seq_len))) return rc;
    const size_t kvw = static_cast<size_t>(d.heads) * d.head_dim;
    char* buf = nullptr;
    const size_t o_out = 0, o_k = align_up(d.hidden * 2, 256), o_v = o_k + align_up(kvw * 2, 256);
    const size_t o_desc = o_v + align_up(kvw * 2, 256);
    CF_CUDA(cudaMalloc(&buf, o_desc + sizeof(LayerDesc)));
    CF_CUDA(cudaMemset(buf, 0, o_desc + sizeof(LayerDesc)));
    ctx.out = reinterpret_cast<__half*>(buf + o_out);
    ctx.k_new = reinterpret_cast<__half*>(buf + o_k);
    ctx.v_new = reinterpret_cast<__half*>(buf + o_v);
    ctx.dev = reinterpret_cast<LayerDesc*>(buf + o_desc);
    ctx.dirty = true;
    std::lock_guard<std::mutex> lk(g_mu);
    auto key = std::make_pair(model, context_id);
    auto it = ds->contexts.find(key);
    if (it != ds->contexts.end()) {  // re-creating an id replaces it, as the reference's map assignment does
        cudaDeviceSynchronize();
        cudaFree(it->second.out);
        ds->contexts.erase(it);
    }
    ds->contexts[key] = ctx;
    return CF_OK;
}

int cf_pythia_graph_set_device_state(int model, int64_t context_id, const int* seq_len_dev, const float* cos_table,
                                     const float* sin_table, int64_t table_stride) {
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = ds->contexts.find(std::make_pair(model, context_id));
    if (it == ds->contexts.end())
        return fail(CF_ERR_INVALID, "Context not initialized. Call create_graph_context first. (id %lld)", (long long)context_id);
    if ((cos_table == nullptr) != (sin_table == nullptr)) return fail(CF_ERR_INVALID, "cos/sin tables must both be set");
    if (cos_table && table_stride <= 0) return fail(CF_ERR_INVALID, "table_stride %lld", (long long)table_stride);
    it->second.seq_dev = seq_len_dev;
    it->second.cos_t = cos_table;
    it->second.sin_t = sin_table;
    it->second.table_stride = static_cast<int>(table_stride);
    return CF_OK;
}

int cf_pythia_graph_decode_step(int model, int64_t context_id, const CfStepArgs* a, int64_t seq_len, void* stream,
                                void** output, void** k_new, void** v_new) {
    CfDims d;
    int rc = model_dims(model, &d);
    if (rc) return rc;
    if (!a) return fail(CF_ERR_INVALID, "null step args");
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    GraphCtx* ctx;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = ds->contexts.find(std::make_pair(model, context_id));
        if (it == ds->contexts.end())
            return fail(CF_ERR_INVALID, "Context not initialized. Call create_graph_context first. (id %lld)", (long long)context_id);
        ctx = &it->second;
    }
    if (!a->input || !a->ln_weight || !a->ln_bias || !a->qkv_bias || !a->o_bias || !a->post_ln_weight ||
        !a->post_ln_bias || !a->mlp_up_bias || !a->mlp_down_bias)
        return fail(CF_ERR_INVALID, "null pointer in step args");
    if ((a->k_cache && a->k_cache != ctx->host.k_cache) || (a->v_cache && a->v_cache != ctx->host.v_cache))
        return fail(CF_ERR_INVALID, "k_cache / v_cache differ from the tensors the context was created with");
    const bool dev_state = ctx->seq_dev != nullptr;
    if (!dev_state) {
        if (!a->cos || !a->sin) return fail(CF_ERR_INVALID, "null cos/sin");
        if (seq_len < 0 || seq_len >= ctx->host.kv_rows)
            return fail(CF_ERR_INVALID, "current_seq_len %lld outside [0, max_seq_len=%d)", (long long)seq_len, ctx->host.kv_rows);
    }
    LayerDesc& L = ctx->host;
    const __half* np[8] = {static_cast<const __half*>(a->ln_weight),      static_cast<const __half*>(a->ln_bias),
                           static_cast<const __half*>(a->post_ln_weight), static_cast<const __half*>(a->post_ln_bias),
                           static_cast<const __half*>(a->qkv_bias),       static_cast<const __half*>(a->mlp_up_bias),
                           static_cast<const __half*>(a->o_bias),         static_cast<const __half*>(a->mlp_down_bias)};
    const __half** cur[8] = {&L.ln_w, &L.ln_b, &L.pln_w, &L.pln_b, &L.b_qkv, &L.b_up, &L.b_o, &L.b_down};
    for (int i = 0; i < 8; ++i)
        if (*cur[i] != np[i]) {
            *cur[i] = np[i];
            ctx->dirty = true;
        }
    if (ctx->dirty) {
        // first step of a context (or new small tensors): not capturable, like any upload
        if ((rc = refuse_upload_in_capture(st, "graph_decode_step"))) return rc;
        CF_CUDA(cudaMemcpyAsync(ctx->dev, &ctx->host, sizeof(LayerDesc), cudaMemcpyHostToDevice, st));
        ctx->dirty = false;
    }
    Params p;
    base_params(p, d, ds->ws);
    p.layers = ctx->dev;
    p.n_layers = 1;
    p.phase_mask = PH_P1 | PH_P2 | PH_P3;
    p.p3_flags = F3_FULL;
    p.x_in = static_cast<const __half*>(a->input);
    p.out = ctx->out;
    p.k_new = ctx->k_new;
    p.v_new = ctx->v_new;
    if (dev_state) {
        p.seq_ptr = ctx->seq_dev;
        if (ctx->cos_t) {
            p.cos = ctx->cos_t;
            p.sin = ctx->sin_t;
            p.rope_stride = ctx->table_stride;
        } else {
            p.cos = a->cos;
            p.sin = a->sin;
        }
    } else {
        p.cos = a->cos;
        p.sin = a->sin;
        p.seq_host = static_cast<int>(seq_len);
    }
    if ((rc = launch(*ds, d, p, st))) return rc;
    if (output) *output = ctx->out;
    if (k_new) *k_new = ctx->k_new;
    if (v_new) *v_new = ctx->v_new;
    return CF_OK;
}

int cf_pythia_destroy_graph_context(int model, int64_t context_id) {
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    std::lock_guard<std::mutex> lk(g_mu);
    auto it = ds->contexts.find(std::make_pair(model, context_id));
    if (it == ds->contexts.end()) return CF_OK;  // erase of a missing key is a no-op in the reference too
    CF_CUDA(cudaDeviceSynchronize());
    cudaFree(it->second.out);
    ds->contexts.erase(it);
    return CF_OK;
}

// ----------------------------------------------------------------------------- decoder
int cf_decoder_create(const CfDecoderConfig* cfg, int64_t* handle) {
    if (!cfg || !handle) return fail(CF_ERR_INVALID, "null argument");
    int rc = check_dims(cfg->dims);
    if (rc) return rc;
    if (cfg->n_layers <= 0 || cfg->n_layers > 1024) return fail(CF_ERR_INVALID, "n_layers %d", cfg->n_layers);
    if (cfg->max_seq_len <= 0 || cfg->max_seq_len > 0x7fffffff) return fail(CF_ERR_INVALID, "max_seq_len");
    if (cfg->tp_size < 1 || cfg->tp_rank < 0 || cfg->tp_rank >= cfg->tp_size) return fail(CF_ERR_INVALID, "tp rank/size");
    if (!cfg->cos_table || !cfg->sin_table) return fail(CF_ERR_INVALID, "null rope table");
    if (cfg->dims.vocab < 0 || (cfg->dims.vocab % GRAN) != 0) return fail(CF_ERR_INVALID, "vocab %d must be a multiple of %d", cfg->dims.vocab, GRAN);
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    Decoder* dc = new Decoder();
    dc->cfg = *cfg;
    dc->dev = ds->dev;
    dc->layers_h.resize(cfg->n_layers);
    dc->layer_set.assign(cfg->n_layers, false);
    if ((rc = ws_alloc(dc->ws))) {
        delete dc;
        return rc;
    }
    const size_t H2 = align_up(static_cast<size_t>(cfg->dims.hidden) * 2, 256);
    const size_t o_tok = 0, o_seq = 256, o_hid = 512, o_h0 = o_hid + H2, o_h1 = o_h0 + H2, o_part = o_h1 + H2;
    const size_t o_log = o_part + H2;
    const size_t o_desc = align_up(o_log + sizeof(float) * (cfg->dims.vocab > 0 ? cfg->dims.vocab : 1), 256);
    const size_t o_tail = o_desc + sizeof(LayerDesc) * cfg->n_layers;
    const size_t total = o_tail + sizeof(TailDesc);
    char* b = nullptr;
    cudaError_t e = cudaMalloc(&b, total);
    if (e != cudaSuccess) {
        cudaFree(dc->ws.base);
        delete dc;
        return fail(CF_ERR_CUDA, "cudaMalloc failed: %s", cudaGetErrorString(e));
    }
    cudaMemset(b, 0, total);
    dc->token_d = reinterpret_cast<int*>(b + o_tok);
    dc->seq_d = reinterpret_cast<int*>(b + o_seq);
    dc->hidden_d = reinterpret_cast<__half*>(b + o_hid);
    dc->hid0 = reinterpret_cast<__half*>(b + o_h0);
    dc->hid1 = reinterpret_cast<__half*>(b + o_h1);
    dc->partial_d = reinterpret_cast<__half*>(b + o_part);
    dc->logits_d = reinterpret_cast<float*>(b + o_log);
    dc->layers_d = reinterpret_cast<LayerDesc*>(b + o_desc);
    dc->tail_d = reinterpret_cast<TailDesc*>(b + o_tail);
    std::lock_guard<std::mutex> lk(g_mu);
    *handle = g_next_handle++;
    g_decoders[*handle] = dc;
    return CF_OK;
}

int cf_decoder_set_layer(int64_t handle, int layer, const CfLayerWeights* w, void* k_cache, void* v_cache) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (layer < 0 || layer >= dc->cfg.n_layers) return fail(CF_ERR_INVALID, "layer %d", layer);
    if (!w || !k_cache || !v_cache) return fail(CF_ERR_INVALID, "null argument");
    if (!w->qkv_weight || !w->qkv_bias || !w->o_weight || !w->o_bias || !w->ln_weight || !w->ln_bias ||
        !w->post_ln_weight || !w->post_ln_bias || !w->mlp_up_weight || !w->mlp_up_bias || !w->mlp_down_weight ||
        !w->mlp_down_bias)
        return fail(CF_ERR_INVALID, "null weight pointer");
    if ((rc = build_layer_desc(dc->layers_h[layer], dc->cfg.dims, *w, k_cache, v_cache, dc->cfg.max_seq_len))) return rc;
    dc->layer_set[layer] = true;
    dc->finalized = false;
    return CF_OK;
}

int cf_decoder_set_head(int64_t handle, const CfHeadWeights* head) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!head || !head->embed_in || !head->final_ln_weight || !head->final_ln_bias || !head->embed_out)
        return fail(CF_ERR_INVALID, "null head pointer");
    if (dc->cfg.dims.vocab <= 0) return fail(CF_ERR_INVALID, "decoder was created with vocab 0");
    memset(&dc->tail_h, 0, sizeof(TailDesc));
    if ((rc = encode_weight(&dc->tail_h.tm_head, head->embed_out, dc->cfg.dims.hidden, dc->cfg.dims.vocab))) return rc;
    dc->tail_h.fln_w = static_cast<const __half*>(head->final_ln_weight);
    dc->tail_h.fln_b = static_cast<const __half*>(head->final_ln_bias);
    dc->tail_h.vocab = dc->cfg.dims.vocab;
    dc->head = *head;
    dc->head_set = true;
    dc->finalized = false;
    return CF_OK;
}

int cf_decoder_finalize(int64_t handle) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    for (int l = 0; l < dc->cfg.n_layers; ++l)
        if (!dc->layer_set[l]) return fail(CF_ERR_INVALID, "layer %d was never set", l);
    if (!dc->head_set) return fail(CF_ERR_INVALID, "head weights were never set");
    CF_CUDA(cudaMemcpy(dc->layers_d, dc->layers_h.data(), sizeof(LayerDesc) * dc->cfg.n_layers, cudaMemcpyHostToDevice));
    CF_CUDA(cudaMemcpy(dc->tail_d, &dc->tail_h, sizeof(TailDesc), cudaMemcpyHostToDevice));
    dc->finalized = true;
    return CF_OK;
}

int cf_decoder_state(int64_t handle, int** token, int** seq_len, float** logits, void** hidden, void** partial,
                     float** shard_max, int** shard_idx) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (token) *token = dc->token_d;
    if (seq_len) *seq_len = dc->seq_d;
    if (logits) *logits = dc->logits_d;
    if (hidden) *hidden = dc->hidden_d;
    if (partial) *partial = dc->partial_d;
    if (shard_max) *shard_max = dc->ws.amax_val;
    if (shard_idx) *shard_idx = dc->ws.amax_idx;
    return CF_OK;
}

int cf_decoder_tp_export(int64_t handle, void* ipc_handle_out) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!ipc_handle_out) return fail(CF_ERR_INVALID, "null handle buffer");
    if (dc->cfg.tp_size < 2 || dc->cfg.tp_size > MAX_TP) return fail(CF_ERR_INVALID, "tp_size %d (2..%d)", dc->cfg.tp_size, MAX_TP);
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    if ((rc = pick_cfg(*ds, dc->cfg.dims.head_dim))) return rc;
    if (!dc->tp_local) {
        const TpLayout tl{dc->cfg.dims.hidden, dc->cfg.tp_size};  // zero-filled: epoch 0 means never written
        const size_t bytes = align_up(tl.bytes(), 256) + 256;
        CF_CUDA(cudaMalloc(&dc->tp_local, bytes));
        CF_CUDA(cudaMemset(dc->tp_local, 0, bytes));
        dc->tp_count = reinterpret_cast<unsigned*>(dc->tp_local + align_up(tl.bytes(), 256));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    CF_CUDA(cudaIpcGetMemHandle(&h, dc->tp_local));
    memcpy(ipc_handle_out, &h, sizeof(h));
    return CF_OK;
}

int cf_decoder_tp_connect(int64_t handle, const void* all_handles) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!all_handles) return fail(CF_ERR_INVALID, "null handles");
    if (!dc->tp_local) return fail(CF_ERR_INVALID, "call cf_decoder_tp_export first");
    if (dc->tp_connected) return CF_OK;
    for (int r = 0; r < dc->cfg.tp_size; ++r) {
        if (r == dc->cfg.tp_rank) {
            dc->tp_peer[r] = dc->tp_local;
            continue;
        }
        cudaIpcMemHandle_t h;
        memcpy(&h, static_cast<const char*>(all_handles) + 64 * r, sizeof(h));
        void* ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess)
            return fail(CF_ERR_CUDA, "cudaIpcOpenMemHandle for rank %d failed: %s (peer access over NVLink is required)", r,
                        cudaGetErrorString(e));
        dc->tp_peer[r] = static_cast<unsigned char*>(ptr);
        dc->tp_ipc = true;
    }
    dc->tp_connected = true;
    return CF_OK;
}

int cf_decoder_tp_connect_pointers(int64_t handle, void* const* peer_buffers) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!peer_buffers) return fail(CF_ERR_INVALID, "null pointer table");
    if (!dc->tp_local) return fail(CF_ERR_INVALID, "call cf_decoder_tp_export first");
    for (int r = 0; r < dc->cfg.tp_size; ++r) {
        if (r == dc->cfg.tp_rank) {
            dc->tp_peer[r] = dc->tp_local;
        } else {
            if (!peer_buffers[r]) return fail(CF_ERR_INVALID, "null buffer for rank %d", r);
            if (reinterpret_cast<uintptr_t>(peer_buffers[r]) & 15) return fail(CF_ERR_INVALID, "buffer of rank %d not 16-byte aligned", r);
            dc->tp_peer[r] = static_cast<unsigned char*>(peer_buffers[r]);
        }
    }
    dc->tp_connected = true;
    return CF_OK;
}

int cf_decoder_tp_buffer(int64_t handle, void** buffer, int64_t* bytes) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!dc->tp_local) return fail(CF_ERR_INVALID, "call cf_decoder_tp_export first");
    if (buffer) *buffer = dc->tp_local;
    if (bytes) *bytes = static_cast<int64_t>(TpLayout{dc->cfg.dims.hidden, dc->cfg.tp_size}.bytes());
    return CF_OK;
}

int cf_decoder_step(int64_t handle, void* stream) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!dc->finalized) return fail(CF_ERR_INVALID, "decoder not finalized");
    if (dc->cfg.tp_size != 1 && !dc->tp_connected)
        return fail(CF_ERR_INVALID, "tensor-parallel decoder: exchange buffers not connected (cf_decoder_tp_export / cf_decoder_tp_connect), or use the layer_partial/finish/tail calls");
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    Params p;
    decoder_params(*dc, p);
    if (dc->cfg.tp_size > 1) {
        p.tp_size = dc->cfg.tp_size;
        p.tp_rank = dc->cfg.tp_rank;
        for (int r = 0; r < dc->cfg.tp_size; ++r) p.tp_peer[r] = dc->tp_peer[r];
        p.tp_epoch_base = dc->tp_count;
        // experiment switch (must be equal on every rank): no difference measured at 2 GPUs, so off
        p.tp_packed = env_int("CFB200_TP_PACKED", 0) != 0;
    }
    p.layers = dc->layers_d;
    p.tail = dc->tail_d;
    p.n_layers = dc->cfg.n_layers;
    p.phase_mask = PH_P1 | PH_P2 | PH_P3 | PH_P4;
    p.p3_flags = F3_FULL;
    p.embed = static_cast<const __half*>(dc->head.embed_in);
    p.token_in = dc->token_d;
    p.out = dc->hidden_d;
    p.logits = dc->logits_d;
    p.token_out = dc->token_d;
    p.seq_inc = dc->seq_d;
    p.vocab_offset = dc->head.vocab_offset;
    return launch(*ds, dc->cfg.dims, p, static_cast<cudaStream_t>(stream));
}

int cf_decoder_layer_partial(int64_t handle, int layer, void* stream) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!dc->finalized) return fail(CF_ERR_INVALID, "decoder not finalized");
    if (layer < 0 || layer >= dc->cfg.n_layers) return fail(CF_ERR_INVALID, "layer %d", layer);
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int H = dc->cfg.dims.hidden;
    if (layer == 0) {
        embed_gather_kernel<<<4, 256, 0, st>>>(static_cast<const __half*>(dc->head.embed_in), dc->token_d, dc->hid1, H);
        CF_CUDA(cudaGetLastError());
    }
    Params p;
    decoder_params(*dc, p);
    p.layers = dc->layers_d + layer;
    p.n_layers = 1;
    p.phase_mask = PH_P1 | PH_P2 | PH_P3;
    p.p3_flags = F3_USE_O | F3_USE_DOWN;
    // hidden state ping-pong: layer l reads hid[(l+1)&1], layer_finish writes hid[l&1]
    p.x_in = (layer & 1) ? dc->hid0 : dc->hid1;
    p.out = dc->partial_d;
    return launch(*ds, dc->cfg.dims, p, st);
}

int cf_decoder_layer_finish(int64_t handle, int layer, void* stream) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (layer < 0 || layer >= dc->cfg.n_layers) return fail(CF_ERR_INVALID, "layer %d", layer);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const LayerDesc& L = dc->layers_h[layer];
    const __half* x = (layer & 1) ? dc->hid0 : dc->hid1;
    __half* y = (layer == dc->cfg.n_layers - 1) ? dc->hidden_d : ((layer & 1) ? dc->hid1 : dc->hid0);
    tp_finish_kernel<<<4, 256, 0, st>>>(x, dc->partial_d, L.b_o, L.b_down, y, dc->cfg.dims.hidden);
    CF_CUDA(cudaGetLastError());
    return CF_OK;
}

int cf_decoder_tail(int64_t handle, void* stream) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!dc->finalized) return fail(CF_ERR_INVALID, "decoder not finalized");
    DeviceState* ds;
    if ((rc = get_device(&ds))) return rc;
    Params p;
    decoder_params(*dc, p);
    p.tail = dc->tail_d;
    p.n_layers = 0;
    p.phase_mask = PH_P4;
    p.x_in = dc->hidden_d;
    p.logits = dc->logits_d;
    p.vocab_offset = dc->head.vocab_offset;
    return launch(*ds, dc->cfg.dims, p, static_cast<cudaStream_t>(stream));
}

int cf_decoder_select_token(int64_t handle, const float* pairs_val, const int* pairs_idx, void* stream) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!pairs_val || !pairs_idx) return fail(CF_ERR_INVALID, "null pointer");
    select_token_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(pairs_val, pairs_idx, dc->cfg.tp_size,
                                                                        dc->token_d, dc->seq_d);
    CF_CUDA(cudaGetLastError());
    return CF_OK;
}

int cf_decoder_status(int64_t handle, int* status) {
    Decoder* dc;
    int rc = find_decoder(handle, &dc);
    if (rc) return rc;
    if (!status) return fail(CF_ERR_INVALID, "null status");
    // a blocking 4-byte read: it waits for the work queued before it on the legacy default stream
    // (and the streams that synchronise with it); callers on other streams synchronise first
    CF_CUDA(cudaMemcpy(status, dc->ws.status, sizeof(int), cudaMemcpyDeviceToHost));
    return CF_OK;
}

int cf_debug_noalloc_scratch(void** base, int64_t* bytes, int64_t* status_offset) {
    std::lock_guard<std::mutex> lk(g_noalloc_mu);
    NoAllocDevice* nd;
    int rc = noalloc_setup(&nd);
    if (rc) return rc;
    if (base) *base = nd->scratch;
    if (bytes) *bytes = static_cast<int64_t>(NOALLOC_SCRATCH_BYTES);
    if (status_offset) *status_offset = static_cast<int64_t>(NA_OFF_SYNC + 16);
    return CF_OK;
}

int cf_decoder_destroy(int64_t handle) {
    Decoder* dc = nullptr;
    {
        std::lock_guard<std::mutex> lk(g_mu);
        auto it = g_decoders.find(handle);
        if (it == g_decoders.end()) return CF_OK;
        dc = it->second;
        g_decoders.erase(it);
    }
    cudaDeviceSynchronize();
    if (dc->tp_ipc)
        for (int r = 0; r < MAX_TP; ++r)
            if (dc->tp_peer[r] && dc->tp_peer[r] != dc->tp_local) cudaIpcCloseMemHandle(dc->tp_peer[r]);
    if (dc->tp_local) cudaFree(dc->tp_local);
    cudaFree(dc->token_d);
    cudaFree(dc->ws.base);
    delete dc;
    return CF_OK;
}

int cf_prefill_linear(const void* x, const void* weight, const void* bias, const void* residual, void* out,
                      int64_t m, int64_t n, int64_t k, int act, void* stream) {
    if (!x || !weight || !out) return fail(CF_ERR_INVALID, "null argument");
    if (m <= 0 || n <= 0 || k <= 0 || m > 0x7fffffff || n > 0x7fffffff || k > 0x7fffffff)
        return fail(CF_ERR_INVALID, "bad GEMM extent %lld x %lld x %lld", (long long)m, (long long)n, (long long)k);
    if ((n % 8) || (k % 8)) return fail(CF_ERR_UNSUPPORTED, "n (%lld) and k (%lld) must be multiples of 8", (long long)n, (long long)k);
    if (act != CF_ACT_NONE && act != CF_ACT_GELU_TANH && act != CF_ACT_GELU_ERF) return fail(CF_ERR_INVALID, "activation %d", act);
    if (residual && act != CF_ACT_NONE) return fail(CF_ERR_INVALID, "a residual goes with CF_ACT_NONE only");
    DeviceState* ds;
    int rc = get_device(&ds);
    if (rc) return rc;
    const char* msg = prefill_linear(x, weight, bias, residual, out, static_cast<int>(m), static_cast<int>(n),
                                     static_cast<int>(k), act, static_cast<cudaStream_t>(stream));
    if (msg) return fail(CF_ERR_CUDA, "prefill GEMM: %s", msg);
    return CF_OK;
}

}  // extern "C"
