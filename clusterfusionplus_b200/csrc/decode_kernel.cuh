// Fused GPT-NeoX/Pythia decode step (batch 1) for sm_100a: one persistent,
// co-resident grid that streams every weight and KV byte exactly once through a
// TMA ring and keeps all reductions in fp32 and in a fixed order.
//
// It covers what the reference does in Pythia6b9DecoderLayerKernel
// (include/5090/pythia_6b9/kernel.cuh:56-900) and PythiaDecoderLayerKernel
// (include/5090/pythia_2b8/kernel.cuh:51-950), its split variants
// (pythia_2b8/kernel_attention.cuh:51, kernel_mlp.cuh:29) and the decode-loop
// tail the reference leaves to PyTorch (tests/benchmark_decode_6b9.py:186-195),
// but is organised differently:
//
//   P1  LayerNorm (both norms share mean/rstd) -> {QKV, MLP-up} GEMV, output rows
//       partitioned over ALL CTAs (no split-K), + bias (+ GELU for MLP-up)
//   P2  partial NeoX RoPE, KV append, flash-decode over (head, 128-row chunk)
//       items spread evenly over all CTAs, per-CTA partial (m, l, acc) in fp32
//   P3  merge attention partials, {O-proj, MLP-down} as ONE GEMV over
//       K = [attn ; mid]; K-chunks interleaved over the CTAs of a cluster and
//       the partial rows summed through distributed shared memory
//       (dsm.cuh), + biases + residual -> fp16 output
//   P4  (optional tail) final LayerNorm -> LM-head GEMV -> argmax
//
// There is no grid barrier between the phases of a layer nor between layers: what
// one CTA hands to the others travels as epoch-tagged words or epoch-stamped records
// that the readers poll (st_ll / publish_record below), and the MLP intermediate is
// gated by a count of CTAs past P1.  Grid barriers remain in the tail only.
//
// One producer thread issues every TMA load of the whole launch in program
// order, limited only by ring capacity: it runs ahead of the consumers across
// phase and layer boundaries, so the next phase's weights are already landing
// while the consumers wait for other CTAs' data.
//
// Determinism: no atomics on data; every sum has a fixed association order that
// depends only on (grid size, cluster size, sequence length).
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "dsm.cuh"
#include "pipeline.cuh"

namespace cfb {

constexpr int KCHUNK = 256;                 // K elements per TMA box (512 B rows)
constexpr int GRAN = 8;                     // rows per granule (one box = 8 x 256 fp16 = 4 KB)
constexpr int SLOT_BYTES = GRAN * KCHUNK * 2;
constexpr int NSLOT = 9;                    // granules per stage (warps 0..7 take slot w, warp 0 also slot 8)
constexpr int STAGE_BYTES = NSLOT * SLOT_BYTES;  // 36 KB
constexpr int MAX_STAGES = 8;
constexpr int NCWARP = 8;                   // consumer warps
constexpr int NCTHR = NCWARP * 32;          // consumer threads
constexpr int NHWARP = 3;                   // helper warps: latency-bound side work off the consumers' path
constexpr int NHTHR = NHWARP * 32;
constexpr int NTHREADS = NCTHR + 32 + NHTHR;  // consumers + producer warp + helpers = 12 warps (register-file granule)
constexpr int KV_TILE = 128;                // cache rows per attention item (K tile and V tile are separate stages)
constexpr int KV_RPH = KV_TILE / (2 * NCWARP);  // rows per half-warp per item
constexpr int MAXL = 4;                     // attention partial slots per CTA
constexpr int MAXHPC = 2;                   // heads one CTA's attention items can span (items per CTA <= chunks per head)
constexpr int NFWARP = 2;                   // helper warps that finish attention partials (helper warps 1 .. NFWARP)
constexpr int NFTHR = NFWARP * 32;
constexpr int MAX_P3_ROWS = 128;            // output rows one cluster may own in P3
constexpr int MAX_H = 4096;                 // LayerNorm register staging limit
constexpr int WTS_SLOTS = 256;              // (attention chunk, head, partial) merge weights one CTA may need
constexpr int MAX_PARTS = 64;               // partials one head may be split into
constexpr int MAX_TP = 8;                   // ranks of a tensor-parallel group

enum : int { PH_P1 = 1, PH_P2 = 2, PH_P3 = 4, PH_P4 = 8 };
// variants of the layer for the Llama attention block (reference: include/5090/llama/kernel_sglang.cuh)
enum : int {
    AF_RMS_ADD = 1,     // norm = RMSNorm(x + residual) with weight only; the sum is also an output
    AF_QKV_PLANAR = 2,  // QKV weight rows are [Q of all heads; K of all heads; V of all heads]
    AF_NO_APPEND = 4,   // the caches hold exactly seq_len rows and are not written
    AF_GELU_ERF = 8,    // MLP activation is the exact GELU x * Phi(x) instead of the tanh form
    AF_NO_QKV = 16,     // P1 streams the MLP-up matrix only (an MLP block on its own)
    AF_SWIGLU = 32,     // the up matrix is [gate rows; up rows] (F_up = 2F, no bias); mid = silu(gate) * up
};
enum : int {
    F3_USE_O = 1,       // include W_o chunks (attention output) in P3
    F3_USE_DOWN = 2,    // include W_down chunks (MLP) in P3
    F3_ADD_X = 4,       // + residual input
    F3_ADD_BO = 8,      // + o-proj bias
    F3_ADD_BDOWN = 16,  // + mlp-down bias
    F3_MID_F16 = 32,    // MLP intermediate comes from an fp16 tensor instead of fp32 scratch
};

// Per-layer descriptor, resident in device memory.
// A weight matrix is described five times, with boxes of 8, 16, 24, 32 and 64 rows (x 256 K elements):
// a stage's run of up to 9 consecutive granules is fetched with at most two TMA operations (the copy engine
// takes them one at a time, a fraction of a microsecond each, so their number matters as much as their bytes).
struct WeightMaps {
    CUtensorMap r8, r16, r24, r32, r64;
};

struct alignas(128) LayerDesc {
    WeightMaps tm_qkv, tm_up, tm_o, tm_down;
    CUtensorMap tm_k, tm_v;
    const __half *ln_w, *ln_b, *pln_w, *pln_b;
    const __half *b_qkv, *b_up, *b_o, *b_down;
    __half *k_cache, *v_cache;
    int kv_rows;  // rows in the cache allocation
    int pad_[7];
};

struct alignas(128) TailDesc {
    WeightMaps tm_head;
    const __half *fln_w, *fln_b;
    int vocab;
    int pad_[11];
};

struct Params {
    const LayerDesc* layers;
    const TailDesc* tail;
    int n_layers;
    int H;         // hidden size (K of P1, rows of P3)
    int NH;        // heads held by this rank
    int R;         // rotary dims
    int F;         // MLP intermediate width held by this rank
    int phase_mask;
    int p3_flags;
    int nstage;
    int xbuf_floats;
    int aux_off;       // floats into xbuf: [MAXHPC][3][D] pre-staged q / new k / new v, then the partial hand-over buffer
    // activations
    const __half* x_in;   // [H]; ignored when embed != nullptr
    const __half* embed;  // optional [V, H] table: x = embed[*token_in]
    const int* token_in;
    __half* out;          // output of the last layer of this launch
    uint2* hid_ll[2];     // hidden state between layers of one launch, ping-pong, {fp16 bits, epoch} per element
    __half* k_new;        // optional [NH*D] (single-layer launches)
    __half* v_new;
    const float* cos;     // row for this position, or table base when rope_stride > 0
    const float* sin;
    int rope_stride;      // floats between table rows; 0 = cos/sin point at the row itself
    int seq_host;         // used when seq_ptr == nullptr
    const int* seq_ptr;   // device-resident sequence length (graph replay)
    // split-API tensors
    __half* mid_f16_out;          // optional fp16 copy of the MLP intermediate
    const __half* mid_f16_in;     // with F3_MID_F16
    const __half* extra_add_f16;  // optional [H] added in the P3 epilogue
    // scratch
    uint2* qkv_ll;     // [3*NH*D] {fp32 bits, epoch}: q/k/v rows travel with the epoch of their launch and layer
    unsigned* epoch_base;    // running base of those epochs; the last CTA out adds (layers + 2)
    int qkv_any_epoch; // the launch has no P1: take whatever an earlier launch left in qkv_ll
    float* mid_f32;    // [F]
    float* attn_part;  // [grid][MAXL][D+4]: D numerators, max, denominator, epoch (written last), 1 pad
    float* attn_new;   // [NH][D+4], same record
    int part_any_epoch;  // the launch has no P2: take the attention partials an earlier launch left
    unsigned* sync;    // [0] barrier count, [1] exit count, [2] epoch base, [3] CTAs past P1 (counts up over layers)
    int* status;
    // tail outputs
    float* logits;     // optional [vocab]
    float* amax_val;   // [grid]
    int* amax_idx;     // [grid]
    int* token_out;    // next token id (may alias token_in)
    int* seq_inc;      // optional: *seq_inc += 1 at the end of the launch
    int vocab_offset;  // added to the argmax index (vocabulary shards)
    int p1_joint;      // P1 row split: 1 = every CTA QKV share then up share, jointly balanced (host verified it
                       // is monotone), 0 = the same with independent even splits, 2 = grouped (QKV CTAs, up CTAs)
    int gq;            // grouped split: CTAs in the QKV group
    int F_up;          // rows of the MLP-up matrix when they are not F (AF_SWIGLU: 2F); 0 = F
    int arch_flags;    // AF_*
    float norm_eps;    // RMSNorm epsilon (AF_RMS_ADD)
    const __half* residual_in;  // [H], AF_RMS_ADD
    __half* residual_out;       // [H], AF_RMS_ADD: x + residual (must not alias residual_in)
    // optional timeline: [grid][n_layers + 1][TRACE_EVENTS] globaltimer stamps (diagnostics)
    unsigned long long* trace;
    int touch_only;    // diagnostics: row-GEMV consumers take and release the stages without the arithmetic
    // tensor-parallel exchange over peer memory (tp_size > 1): every rank owns one buffer laid
    // out as TpLayout; tp_peer[r] is rank r's buffer as mapped into this process.
    int tp_size, tp_rank;
    unsigned char* tp_peer[MAX_TP];
    unsigned* tp_epoch_base;    // two local words: [0] running epoch base of the exchanges, [1] launches so far
    int tp_packed;     // exchange words of one CTA are contiguous (its threads' peer stores coalesce) instead of row-indexed
    // Launched with programmatic stream serialization: this grid may start while the kernel before it in the
    // stream is still draining.  Weights are never written on the device, so the producer streams its first
    // ring-full of P1 stages at once; everything else waits for that kernel (griddepcontrol.wait) first.  The
    // caller promises that the preceding kernel writes neither seq_len nor the descriptors.
    int pdl;
    int merge_seg_max;  // diagnostics: > 0 caps the segments a head's partial records are cut into for the merge (1 = never cut)
    // Single-layer launches whose caches change shape from call to call (the Llama block takes caches of exactly
    // seq_len rows): the key / value tensor maps travel in the kernel parameters instead of the layer descriptor,
    // so the descriptor depends on the weights only and nothing is uploaded per call.
    int kv_inline;       // 1: use kv_maps / kv_rows_inline
    int kv_rows_inline;  // rows the inline maps cover
    alignas(64) CUtensorMap kv_maps[2];  // key, value
};

__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Exchange buffer of one rank (H = hidden).  Every word travels with the epoch it belongs
// to in the same aligned 8-byte store (value, epoch), so a reader that sees the epoch has the
// value: no fence and no separate flag, one NVLink crossing of latency.
//   partial[2][tp][H]  {fp32 value, u32 epoch}   slot [epoch parity][source rank]
//   pairs  [2][tp][2]  {bits, u32 epoch}         slot [launch parity][source rank]: max logit, index
struct TpLayout {
    int H, tp;
    __host__ __device__ size_t partial_off(int parity, int src) const { return (static_cast<size_t>(parity) * tp + src) * H * 8; }
    __host__ __device__ size_t pairs_off(int parity, int src) const { return static_cast<size_t>(2) * tp * H * 8 + (static_cast<size_t>(parity) * tp + src) * 16; }
    __host__ __device__ size_t bytes() const { return pairs_off(2, 0); }
};

// pause between re-reads of a word in global memory that has not arrived yet
constexpr int POLL_BACKOFF_NS = 96;

// A tagged word is ONE naturally aligned 64-bit access, {payload bits (low), epoch (high)}: the
// PTX memory model makes an aligned scalar b64 single-copy atomic, so a reader that sees the epoch
// has the payload that was stored with it (a v2.u32 access would formally be two accesses).
// Scope: .gpu for words that stay on this GPU, .sys for words a peer GPU writes or reads.
__device__ __forceinline__ unsigned long long ll_pack(unsigned bits, unsigned epoch) {
    return (static_cast<unsigned long long>(epoch) << 32) | bits;
}
__device__ __forceinline__ uint2 ll_unpack(unsigned long long v) {
    return make_uint2(static_cast<unsigned>(v), static_cast<unsigned>(v >> 32));
}
__device__ __forceinline__ void st_ll(void* p, unsigned bits, unsigned epoch) {
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(ll_pack(bits, epoch)) : "memory");
}
__device__ __forceinline__ void st_ll_sys(void* p, unsigned bits, unsigned epoch) {
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(ll_pack(bits, epoch)) : "memory");
}
__device__ __forceinline__ uint2 ld_ll(const void* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return ll_unpack(v);
}
__device__ __forceinline__ uint2 ld_ll_sys(const void* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.sys.global.b64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return ll_unpack(v);
}
// two adjacent words in one 16-byte load (each b64 element is atomic on its own): {bits0, epoch0, bits1, epoch1}
__device__ __forceinline__ uint4 ld_ll2(const void* p) {
    unsigned long long a, b;
    asm volatile("ld.relaxed.gpu.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
    return make_uint4(static_cast<unsigned>(a), static_cast<unsigned>(a >> 32), static_cast<unsigned>(b),
                      static_cast<unsigned>(b >> 32));
}
// wait (bounded) until the word at p carries `epoch`; returns its payload bits
__device__ __forceinline__ unsigned wait_ll(const void* p, unsigned epoch, const AbortCtl& ab) {
    uint2 v = ld_ll(p);
    if (v.y != epoch) wait_bounded<POLL_BACKOFF_NS>([&] { v = ld_ll(p); return v.y == epoch; }, ab, ST_TIMEOUT_PEER);
    return v.x;
}
__device__ __forceinline__ unsigned wait_ll_sys(const void* p, unsigned epoch, const AbortCtl& ab) {
    uint2 v = ld_ll_sys(p);
    if (v.y != epoch) wait_bounded<POLL_BACKOFF_NS>([&] { v = ld_ll_sys(p); return v.y == epoch; }, ab, ST_TIMEOUT_PEER);
    return v.x;
}

// A record (attention partial) written with plain stores by several threads of the CTA, which
// then met at a CTA barrier: one thread makes them visible device-wide and stamps the record's
// epoch word.  A reader that acquires the epoch sees the record.
__device__ __forceinline__ void publish_record(float* epoch_word, unsigned epoch) {
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(epoch_word), "r"(epoch) : "memory");
}

constexpr int TRACE_EVENTS = 16;
enum : int {
    TR_START = 0, TR_LN_DONE, TR_P1_DONE, TR_BAR1, TR_P2_DONE, TR_BAR2, TR_X3_BUILT, TR_P3_GEMV, TR_P3_DONE,
    TR_PROD_P1 = 10, TR_PROD_P2, TR_PROD_P3,
    TR_MERGE_GO = 13, TR_MERGE_POLLED, TR_MERGE_DONE,  // helper warps: P3's attention merge
};
__device__ __forceinline__ void trace_mark(const Params& p, int cta, int layer, int ev) {
    if (p.trace) p.trace[(static_cast<size_t>(cta) * (p.n_layers + 1) + layer) * TRACE_EVENTS + ev] = globaltimer_ns();
}

__host__ __device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }
// units [part_begin(i), part_begin(i+1)) of `total` belong to part i of `parts`
__host__ __device__ __forceinline__ int part_begin(int i, int total, int parts) {
    return static_cast<int>((static_cast<long long>(i) * total) / parts);
}
// inverse of part_begin: which part owns unit t
__host__ __device__ __forceinline__ int part_of(int t, int total, int parts) {
    return static_cast<int>(((static_cast<long long>(t) + 1) * parts - 1) / total);
}
__host__ __device__ __forceinline__ int head_owner(int h, int NH, int G) { return part_begin(h, G, NH); }

// How a row-partitioned GEMV phase of `cnt` 8-row granules over `KC` K chunks is cut into ring stages.
// A stage has NSLOT slots of (granule, chunk).  With many granules a stage is up to NSLOT granules of ONE
// chunk (m = 1).  With few granules per CTA (small models, tensor-parallel shards) such stages would be
// mostly empty and the phase would be bound by the number of stages, not by bytes; a stage then takes
// n <= 4 granules of m = NSLOT / n consecutive chunks, and the chunk partials of a row are added at the
// end of the round.  Picks the n with the fewest stages (ties: the larger n); returns m, sets n.
__host__ __device__ __forceinline__ int plan_rounds(int cnt, int KC, int& n) {
    n = NSLOT;
    // only where ONE stage per chunk would leave slots empty; with more granules the remainder round of a
    // multi-chunk plan is nearly empty and the plan measured slower (2 GPUs: 1.63 -> 2.12 ms per token)
    if (cnt <= 0 || cnt >= NSLOT) return 1;
    // one chunk per stage unless the alternative needs at most half of the stages: every round of the
    // alternative ends with a reduction between the warps, and at three quarters (6 granules, 4 GPUs) it
    // measured slower (1.15 -> 1.24 ms per token) while at three eighths (3 granules, 8 GPUs) it is faster
    // (1.08 -> 1.01 ms)
    int best = (ceil_div(cnt, NSLOT) * KC) / 2 + 1, m = 1;
    for (int cand = 4; cand >= 1; --cand) {
        const int mm = NSLOT / cand;
        const int stages = ceil_div(cnt, cand) * ceil_div(KC, mm);
        if (stages < best) {
            best = stages;
            n = cand;
            m = mm;
        }
    }
    return m;
}

// ring cursor: same arithmetic on the producer and the consumer side
struct Cursor {
    int stage;
    uint32_t phase;
    int nstage;
    __device__ __forceinline__ void advance() {
        if (++stage == nstage) {
            stage = 0;
            phase ^= 1u;
        }
    }
};

struct Smem {
    uint8_t* ring;
    float* xbuf;
    float* red;     // 64
    float* pm;      // WTS_SLOTS running maxima of the partials this CTA merges
    float* pl;      // WTS_SLOTS their denominators
    int* offs;      // WTS_SLOTS their offsets in the partial buffer (-1: none), fixed for a launch
    float* recv;    // MAX_P3_ROWS
    float* rsum;    // NSLOT * GRAN
    uint64_t* full;
    uint64_t* empty;
    uint64_t* xbar;
    uint64_t* h_go;        // consumers -> helpers: this CTA has entered P3, xbuf's attention chunks are free
    uint64_t* attn_ready;  // helpers -> consumers: merged attention chunks are in xbuf
    uint64_t* mid_ready;   // helper warp 0 -> consumers: every CTA is past P1 and this CTA's MLP chunks are staged in xbuf
    uint64_t* h_layer;     // consumers -> helpers: a new layer has begun, xbuf's spare region is free
    uint64_t* q_ready;     // [MAXHPC] helpers -> consumers: the rotated query of the i-th head this CTA streams is in xbuf
    uint64_t* pf_ready;    // consumers -> helpers: a head's per-warp attention partials are in the hand-over buffer
    uint64_t* pf_free;     // helpers -> consumers: the hand-over buffer has been read
    int* abort_flag;
};

__host__ __device__ __forceinline__ size_t smem_bytes_for(int nstage, int xbuf_floats) {
    return static_cast<size_t>(nstage) * STAGE_BYTES + static_cast<size_t>(xbuf_floats) * 4 +
           (64 + 3 * WTS_SLOTS + MAX_P3_ROWS + NSLOT * GRAN) * 4 + (2 * MAX_STAGES + 9) * 8 + 16;
}

__device__ __forceinline__ Smem carve(uint8_t* base, int nstage, int xbuf_floats) {
    Smem s;
    s.ring = base;
    s.xbuf = reinterpret_cast<float*>(base + static_cast<size_t>(nstage) * STAGE_BYTES);
    s.red = s.xbuf + xbuf_floats;
    s.pm = s.red + 64;
    s.pl = s.pm + WTS_SLOTS;
    s.offs = reinterpret_cast<int*>(s.pl + WTS_SLOTS);
    s.recv = reinterpret_cast<float*>(s.offs + WTS_SLOTS);
    s.rsum = s.recv + MAX_P3_ROWS;
    s.full = reinterpret_cast<uint64_t*>(s.rsum + NSLOT * GRAN);
    s.empty = s.full + MAX_STAGES;
    s.xbar = s.empty + MAX_STAGES;
    s.h_go = s.xbar + 1;
    s.attn_ready = s.xbar + 2;
    s.mid_ready = s.xbar + 3;
    s.h_layer = s.xbar + 4;
    s.q_ready = s.xbar + 5;  // and + 6
    s.pf_ready = s.xbar + 7;
    s.pf_free = s.xbar + 8;
    s.abort_flag = reinterpret_cast<int*>(s.xbar + 9);
    return s;
}

// The auxiliary region of xbuf (Params::aux_off): the pre-staged queries [MAXHPC][3][D] that the helper
// warps write while P1 still runs, then the hand-over buffer of attention partials (one slot per consumer
// warp: D numerators, then NCWARP {max, denominator} pairs).  It lies behind both LayerNorm outputs (live
// through P1) and behind the MLP chunks that P3 stages (written while a partial may still be in the buffer).
// heads whose attention output can fall into one KCHUNK-wide chunk of P3's K range: a whole number when the chunk
// is a multiple of the head width (head_dim 128: two), else the covering count plus one for the straddle (head_dim
// 80: five).  The merge table has one row of partial slots per (chunk, head), so unused rows cost poll iterations.
__host__ __device__ constexpr int heads_per_chunk(int D) { return (KCHUNK % D == 0) ? KCHUNK / D : (KCHUNK + D - 1) / D + 1; }
__host__ __device__ __forceinline__ int aux_floats(int D) { return MAXHPC * 3 * D + NCWARP * D + 2 * NCWARP; }

// ---------------------------------------------------------------- math helpers
__device__ __forceinline__ float gelu_erf_f(float x) { return 0.5f * x * (1.0f + erff(x * 0.7071067811865476f)); }
__device__ __forceinline__ float gelu_tanh_f(float x) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.0f + tanhf(u));
}

// 8 rows x 256 K of one slot against this lane's 8 activations.  The two 16-byte activation reads have a
// 32-byte stride between lanes (two-way bank conflict, 2 of the 34 shared-memory reads of a slot); a layout in
// two planes ([lane][4] twice per chunk) makes them conflict-free but measured 1.3 % slower per token
// (2 500 against 2 467 us, alternating processes on one GPU; larger stack frame), so the plain layout stays.
__device__ __forceinline__ void gemv_slot(const uint8_t* slot, const float* xs, int lane, float (&acc)[GRAN]) {
    const float4 xa = *reinterpret_cast<const float4*>(xs + lane * 8);
    const float4 xb = *reinterpret_cast<const float4*>(xs + lane * 8 + 4);
#pragma unroll
    for (int r = 0; r < GRAN; ++r) {
        const uint4 wv = *reinterpret_cast<const uint4*>(slot + r * (KCHUNK * 2) + lane * 16);
        const float2 w0 = __half22float2(*reinterpret_cast<const __half2*>(&wv.x));
        const float2 w1 = __half22float2(*reinterpret_cast<const __half2*>(&wv.y));
        const float2 w2 = __half22float2(*reinterpret_cast<const __half2*>(&wv.z));
        const float2 w3 = __half22float2(*reinterpret_cast<const __half2*>(&wv.w));
        float a = acc[r];
        a = fmaf(w0.x, xa.x, a);
        a = fmaf(w0.y, xa.y, a);
        a = fmaf(w1.x, xa.z, a);
        a = fmaf(w1.y, xa.w, a);
        a = fmaf(w2.x, xb.x, a);
        a = fmaf(w2.y, xb.y, a);
        a = fmaf(w3.x, xb.z, a);
        a = fmaf(w3.y, xb.w, a);
        acc[r] = a;
    }
}

// Sum 8 per-lane accumulators over the warp with 9 shuffles.  Afterwards lanes
// with (lane & 3) == 0 hold the total of row ((lane>>4)&1)*4 + ((lane>>3)&1)*2 + ((lane>>2)&1).
__device__ __forceinline__ float warp_reduce8(const float (&a)[GRAN], int lane) {
    float b[4], c[2];
    const bool h16 = (lane & 16) != 0, h8 = (lane & 8) != 0, h4 = (lane & 4) != 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float send = h16 ? a[i] : a[i + 4];
        const float keep = h16 ? a[i + 4] : a[i];
        b[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const float send = h8 ? b[i] : b[i + 2];
        const float keep = h8 ? b[i + 2] : b[i];
        c[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
    const float send = h4 ? c[0] : c[1];
    const float keep = h4 ? c[1] : c[0];
    float d = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    d += __shfl_xor_sync(0xffffffffu, d, 2);
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    return d;
}
__device__ __forceinline__ int reduce8_row(int lane) {
    return ((lane >> 4) & 1) * 4 + ((lane >> 3) & 1) * 2 + ((lane >> 2) & 1);
}

// sum over the consumer threads; result broadcast to all of them
__device__ __forceinline__ float block_sum(float v, float* red, int tid) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    consumer_sync(NCTHR);  // red[] free
    if ((tid & 31) == 0) red[tid >> 5] = v;
    consumer_sync(NCTHR);
    float t = 0.f;
#pragma unroll
    for (int i = 0; i < NCWARP; ++i) t += red[i];
    return t;
}

// One q/k/v element from the scratch that P1 filled: wait (bounded) until its word carries this
// layer's epoch.  There is no grid barrier between P1 and P2: a CTA starts on a head as soon
// as that head's rows are there.
struct QkvView {
    const uint2* base;
    unsigned epoch;
    bool any;
    const AbortCtl* ab;
    __device__ __forceinline__ float get(int idx) const {
        if (any) return __uint_as_float(ld_ll(base + idx).x);
        return __uint_as_float(wait_ll(base + idx, epoch, *ab));
    }
};

// rotate-half RoPE on element d (< D) of the head vector starting at scratch index i0
__device__ __forceinline__ float rope_elem(const QkvView& q, int i0, int d, int R, const float* cosr, const float* sinr) {
    const float v = q.get(i0 + d);
    if (d >= R) return v;
    const int half_r = R >> 1;
    const float c = __ldg(cosr + d), s = __ldg(sinr + d);
    const float partner = (d < half_r) ? -q.get(i0 + d + half_r) : q.get(i0 + d - half_r);
    return v * c + partner * s;
}

// ---------------------------------------------------------------- grid barrier
// All consumer threads call it.  Thread 0 publishes this CTA's writes, counts in,
// and spins (bounded) until every CTA of the grid has counted in.
__device__ __forceinline__ void grid_barrier(unsigned* counter, unsigned& epoch, unsigned G, int tid,
                                             const AbortCtl& ab) {
    consumer_sync(NCTHR);
    epoch += 1;
    if (tid == 0) {
        const unsigned target = epoch * G;
        __threadfence();
        atomicAdd(counter, 1u);
        wait_bounded<POLL_BACKOFF_NS>([&] { return ld_acquire_u32(counter) >= target; }, ab, ST_TIMEOUT_GRID);
        __threadfence();
    }
    consumer_sync(NCTHR);
}

// Split form of the same barrier: count in now, wait later.  Work that does not depend on the
// other CTAs goes between the two calls.  All consumer threads call both.
__device__ __forceinline__ void grid_arrive(unsigned* counter, unsigned& epoch, int tid) {
    consumer_sync(NCTHR);
    epoch += 1;
    if (tid == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
    }
}
__device__ __forceinline__ void grid_wait(unsigned* counter, unsigned epoch, unsigned G, int tid, const AbortCtl& ab) {
    if (tid == 0) {
        const unsigned target = epoch * G;
        wait_bounded<POLL_BACKOFF_NS>([&] { return ld_acquire_u32(counter) >= target; }, ab, ST_TIMEOUT_GRID);
        __threadfence();
    }
    consumer_sync(NCTHR);
}

// LayerNorm of x[H] into xbuf (fp32).  which = 0: input norm, 1: post-attention
// norm.  mean/rstd are computed once per layer (two-pass, fp32) and kept in red[32..33].
__device__ __forceinline__ void layer_norm_to_smem(const __half* x, const __half* gamma, const __half* beta, int H,
                                                   float* xbuf, float* red, int tid, bool have_stats) {
    float xv[MAX_H / (NCTHR * 8)][8];
    uint4 graw[MAX_H / (NCTHR * 8)], braw[MAX_H / (NCTHR * 8)];
    const int nvec = H >> 3;
    // gamma / beta do not depend on the statistics: fetch them with x
#pragma unroll
    for (int j = 0; j < MAX_H / (NCTHR * 8); ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
            graw[j] = __ldg(reinterpret_cast<const uint4*>(gamma + v * 8));
            braw[j] = __ldg(reinterpret_cast<const uint4*>(beta + v * 8));
        }
    }
#pragma unroll
    for (int j = 0; j < MAX_H / (NCTHR * 8); ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
            const uint4 raw = ld_cg_u32x4(x + v * 8);
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(h2[k]);
                xv[j][2 * k] = f.x;
                xv[j][2 * k + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) xv[j][k] = 0.f;
        }
    }
    float mean, rstd;
    if (!have_stats) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_H / (NCTHR * 8); ++j)
#pragma unroll
            for (int k = 0; k < 8; ++k) s += xv[j][k];
        mean = block_sum(s, red, tid) / static_cast<float>(H);
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < MAX_H / (NCTHR * 8); ++j) {
            const int v = j * NCTHR + tid;
            if (v < nvec) {
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float d = xv[j][k] - mean;
                    ss = fmaf(d, d, ss);
                }
            }
        }
        const float var = block_sum(ss, red, tid) / static_cast<float>(H);
        rstd = rsqrtf(var + 1e-5f);
        if (tid == 0) {
            red[32] = mean;
            red[33] = rstd;
        }
    } else {
        mean = red[32];
        rstd = red[33];
    }
#pragma unroll
    for (int j = 0; j < MAX_H / (NCTHR * 8); ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
            const __half2* g2 = reinterpret_cast<const __half2*>(&graw[j]);
            const __half2* b2 = reinterpret_cast<const __half2*>(&braw[j]);
            float o[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 g = __half22float2(g2[k]);
                const float2 b = __half22float2(b2[k]);
                o[2 * k] = (xv[j][2 * k] - mean) * rstd * g.x + b.x;
                o[2 * k + 1] = (xv[j][2 * k + 1] - mean) * rstd * g.y + b.y;
            }
            *reinterpret_cast<float4*>(xbuf + v * 8) = make_float4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<float4*>(xbuf + v * 8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
    consumer_sync(NCTHR);
}

// LayerNorm of x[H] into out1 with (gamma1, beta1) and, when out2 != nullptr, into out2 with
// (gamma2, beta2) from the same mean / rstd: the input norm and the post-attention norm of a
// parallel-residual layer see the same input.  Two-pass statistics in fp32.
// The input is either plain fp16 (x) or, when xll != nullptr, the epoch-tagged words another
// layer of this launch produced: they are polled (bounded) until every one carries `xep`,
// which is what replaces a grid barrier between layers.
__device__ __forceinline__ void layer_norm2_to_smem(const __half* x, const uint2* xll, unsigned xep, const AbortCtl& ab,
                                                    const __half* gamma1, const __half* beta1,
                                                    const __half* gamma2, const __half* beta2, int H, float* out1,
                                                    float* out2, float* red, int tid) {
    constexpr int NV = MAX_H / (NCTHR * 8);
    float xv[NV][8];
    uint4 g1[NV], b1[NV], g2[NV], b2[NV];
    const int nvec = H >> 3;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
            g1[j] = __ldg(reinterpret_cast<const uint4*>(gamma1 + v * 8));
            b1[j] = __ldg(reinterpret_cast<const uint4*>(beta1 + v * 8));
            if (out2) {
                g2[j] = __ldg(reinterpret_cast<const uint4*>(gamma2 + v * 8));
                b2[j] = __ldg(reinterpret_cast<const uint4*>(beta2 + v * 8));
            }
        }
    }
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec && xll) {
            uint4 w[4];
            wait_bounded<POLL_BACKOFF_NS>(
                [&] {
                    bool ok = true;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        w[q] = ld_ll2(xll + v * 8 + 2 * q);
                        ok = ok && w[q].y == xep && w[q].w == xep;
                    }
                    return ok;
                },
                ab, ST_TIMEOUT_GRID);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                xv[j][2 * q] = __half2float(__ushort_as_half(static_cast<unsigned short>(w[q].x)));
                xv[j][2 * q + 1] = __half2float(__ushort_as_half(static_cast<unsigned short>(w[q].z)));
            }
        } else if (v < nvec) {
            const uint4 raw = ld_cg_u32x4(x + v * 8);
            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 f = __half22float2(h2[k]);
                xv[j][2 * k] = f.x;
                xv[j][2 * k + 1] = f.y;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) xv[j][k] = 0.f;
        }
    }
    float s = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j)
#pragma unroll
        for (int k = 0; k < 8; ++k) s += xv[j][k];
    const float mean = block_sum(s, red, tid) / static_cast<float>(H);
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                const float d = xv[j][k] - mean;
                ss = fmaf(d, d, ss);
            }
        }
    }
    const float rstd = rsqrtf(block_sum(ss, red, tid) / static_cast<float>(H) + 1e-5f);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
#pragma unroll
            for (int which = 0; which < 2; ++which) {
                if (which == 1 && !out2) break;
                const __half2* gg = reinterpret_cast<const __half2*>(which ? &g2[j] : &g1[j]);
                const __half2* bb = reinterpret_cast<const __half2*>(which ? &b2[j] : &b1[j]);
                float o[8];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const float2 g = __half22float2(gg[k]);
                    const float2 b = __half22float2(bb[k]);
                    o[2 * k] = (xv[j][2 * k] - mean) * rstd * g.x + b.x;
                    o[2 * k + 1] = (xv[j][2 * k + 1] - mean) * rstd * g.y + b.y;
                }
                float* dst = (which ? out2 : out1) + v * 8;
                *reinterpret_cast<float4*>(dst) = make_float4(o[0], o[1], o[2], o[3]);
                *reinterpret_cast<float4*>(dst + 4) = make_float4(o[4], o[5], o[6], o[7]);
            }
        }
    }
    consumer_sync(NCTHR);
}

// RMSNorm of (x + residual) into xbuf (fp32): y = s * rsqrt(mean(s^2) + eps) * gamma, s rounded to
// fp16 first because it is an output of the op (fused add + RMSNorm of the reference:
// include/5090/llama/kernel_sglang.cuh:96-140).  CTA 0 stores s to sum_out.
__device__ __forceinline__ void rms_norm_add_to_smem(const __half* x, const __half* residual, const __half* gamma,
                                                     int H, float eps, float* xbuf, __half* sum_out, float* red,
                                                     int tid) {
    constexpr int NV = MAX_H / (NCTHR * 8);
    float sv[NV][8];
    uint4 graw[NV];
    const int nvec = H >> 3;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) graw[j] = __ldg(reinterpret_cast<const uint4*>(gamma + v * 8));
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
#pragma unroll
        for (int k = 0; k < 8; ++k) sv[j][k] = 0.f;
        if (v < nvec) {
            const uint4 xr = ld_cg_u32x4(x + v * 8);
            uint4 rr = make_uint4(0u, 0u, 0u, 0u);
            if (residual) rr = ld_cg_u32x4(residual + v * 8);
            const __half2* x2 = reinterpret_cast<const __half2*>(&xr);
            const __half2* r2 = reinterpret_cast<const __half2*>(&rr);
            uint4 outraw;
            __half2* o2 = reinterpret_cast<__half2*>(&outraw);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 a = __half22float2(x2[k]), b = __half22float2(r2[k]);
                o2[k] = __floats2half2_rn(a.x + b.x, a.y + b.y);
                const float2 f = __half22float2(o2[k]);
                sv[j][2 * k] = f.x;
                sv[j][2 * k + 1] = f.y;
                ss = fmaf(f.x, f.x, ss);
                ss = fmaf(f.y, f.y, ss);
            }
            if (sum_out) *reinterpret_cast<uint4*>(sum_out + v * 8) = outraw;
        }
    }
    const float rstd = rsqrtf(block_sum(ss, red, tid) / static_cast<float>(H) + eps);
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int v = j * NCTHR + tid;
        if (v < nvec) {
            const __half2* g2 = reinterpret_cast<const __half2*>(&graw[j]);
            float o[8];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float2 g = __half22float2(g2[k]);
                o[2 * k] = sv[j][2 * k] * rstd * g.x;
                o[2 * k + 1] = sv[j][2 * k + 1] * rstd * g.y;
            }
            *reinterpret_cast<float4*>(xbuf + v * 8) = make_float4(o[0], o[1], o[2], o[3]);
            *reinterpret_cast<float4*>(xbuf + v * 8 + 4) = make_float4(o[4], o[5], o[6], o[7]);
        }
    }
    consumer_sync(NCTHR);
}

// ---------------------------------------------------------------- producer side
struct Producer {
    uint32_t ring_addr, full_addr, empty_addr;
    Cursor cur;
    uint64_t policy;
    AbortCtl ab;
    uint32_t issued;  // stages issued so far
    int early_left;   // >= 0: stages that may still be issued before waiting for the preceding kernel (Params::pdl)
    __device__ __forceinline__ bool stop() const { return *ab.flag != 0; }
    __device__ __forceinline__ void depend() {
        if (early_left >= 0) {
            griddep_wait();
            early_left = -1;
        }
    }
    __device__ __forceinline__ void acquire() {
        if (early_left >= 0 && early_left-- == 0) griddep_wait();  // leaves early_left at -1
        mbar_wait(empty_addr + cur.stage * 8, cur.phase ^ 1u, ab, ST_TIMEOUT_EMPTY);
    }
    __device__ __forceinline__ void expect(uint32_t bar, uint32_t bytes) { mbar_arrive_expect_tx(bar, bytes); }
    __device__ __forceinline__ void tile(uint32_t dst, const void* tm, int x, int y, uint32_t bar) {
        tma_load_2d(dst, tm, x, y, bar, policy);
    }
    __device__ __forceinline__ void stage_done() {
        cur.advance();
        ++issued;
    }
    // n consecutive granules starting at granule g0, K offset kx, into consecutive slots at dst:
    // 64-row boxes, then 32-row boxes, then 8-row boxes
    __device__ __forceinline__ void issue_run(const WeightMaps* tm, int kx, int g0, int n, uint32_t dst, uint32_t bar) {
        int w = 0;
        for (; w + 8 <= n; w += 8) tile(dst + w * SLOT_BYTES, &tm->r64, kx, (g0 + w) * GRAN, bar);
        for (; w + 4 <= n; w += 4) tile(dst + w * SLOT_BYTES, &tm->r32, kx, (g0 + w) * GRAN, bar);
        if (n - w == 3) tile(dst + w * SLOT_BYTES, &tm->r24, kx, (g0 + w) * GRAN, bar);
        else if (n - w == 2) tile(dst + w * SLOT_BYTES, &tm->r16, kx, (g0 + w) * GRAN, bar);
        else if (n - w == 1) tile(dst + w * SLOT_BYTES, &tm->r8, kx, (g0 + w) * GRAN, bar);
    }
    // one stage of `n` row granules (rows g0*8 ...) at K offset kx
    __device__ __forceinline__ void rows_stage(const WeightMaps* tm, int kx, int g0, int n) {
        if (stop()) return;
        acquire();
        if (*ab.flag) return;
        const uint32_t bar = full_addr + cur.stage * 8;
        expect(bar, static_cast<uint32_t>(n) * SLOT_BYTES);
        issue_run(tm, kx, g0, n, ring_addr + cur.stage * STAGE_BYTES, bar);
        stage_done();
    }
    // all stages of a row-partitioned GEMV: granules [g0, g0+cnt) of `tm`, KC chunks each
    __device__ __forceinline__ void rows_phase(const WeightMaps* tm, int g0, int cnt, int KC) {
        if (cnt <= 0) return;
        const int nr = ceil_div(cnt, NSLOT), base = cnt / nr, extra = cnt % nr;
        int g = g0;
        for (int r = 0; r < nr; ++r) {
            const int n = base + (r < extra ? 1 : 0);
            for (int c = 0; c < KC; ++c) rows_stage(tm, c * KCHUNK, g, n);
            g += n;
        }
    }
    // Two matrices streamed as ONE sequence of granules (A's cntA granules first, then B's), cut
    // into rounds together, so that a CTA holding a bit of both still runs full-size stages.
    __device__ __forceinline__ void rows_phase2(const WeightMaps* tmA, int gA0, int cntA, const WeightMaps* tmB, int gB0,
                                                int cntB, int KC) {
        const int cnt = cntA + cntB;
        if (cnt <= 0) return;
        int np;
        const int m = plan_rounds(cnt, KC, np);
        if (m > 1) {
            // few granules: stages of np granules x up to m chunks (slot = chunk * n + granule)
            for (int g = 0; g < cnt; g += np) {
                const int n = min(np, cnt - g);
                const int nA = max(0, min(cntA - g, n));
                for (int c0 = 0; c0 < KC; c0 += m) {
                    const int mt = min(m, KC - c0);
                    if (stop()) return;
                    acquire();
                    if (*ab.flag) return;
                    const uint32_t bar = full_addr + cur.stage * 8;
                    expect(bar, static_cast<uint32_t>(n * mt) * SLOT_BYTES);
                    const uint32_t dst = ring_addr + cur.stage * STAGE_BYTES;
                    for (int cc = 0; cc < mt; ++cc) {
                        const uint32_t d = dst + cc * n * SLOT_BYTES;
                        if (nA > 0) issue_run(tmA, (c0 + cc) * KCHUNK, gA0 + g, nA, d, bar);
                        if (n > nA) issue_run(tmB, (c0 + cc) * KCHUNK, gB0 + g + nA - cntA, n - nA, d + nA * SLOT_BYTES, bar);
                    }
                    stage_done();
                }
            }
            return;
        }
        const int nr = ceil_div(cnt, NSLOT), base = cnt / nr, extra = cnt % nr;
        int g = 0;
        for (int r = 0; r < nr; ++r) {
            const int n = base + (r < extra ? 1 : 0);
            const int nA = max(0, min(cntA - g, n));  // granules of this round that belong to A
            for (int c = 0; c < KC; ++c) {
                if (stop()) return;
                acquire();
                if (*ab.flag) return;
                const uint32_t bar = full_addr + cur.stage * 8;
                expect(bar, static_cast<uint32_t>(n) * SLOT_BYTES);
                const uint32_t dst = ring_addr + cur.stage * STAGE_BYTES;
                if (nA > 0) issue_run(tmA, c * KCHUNK, gA0 + g, nA, dst, bar);
                if (n > nA) issue_run(tmB, c * KCHUNK, gB0 + g + nA - cntA, n - nA, dst + nA * SLOT_BYTES, bar);
                stage_done();
            }
            g += n;
        }
    }
    // one attention item = two stages: the K tile, then the V tile of the same 128 rows
    template <int D>
    __device__ __forceinline__ void kv_stage(const CUtensorMap* tmk, const CUtensorMap* tmv, int h, int ch) {
        constexpr uint32_t TILE = KV_TILE * D * 2;
        static_assert(TILE <= STAGE_BYTES, "a K or V tile must fit one ring stage");
#pragma unroll
        for (int kv = 0; kv < 2; ++kv) {
            acquire();
            if (*ab.flag) return;
            const uint32_t bar = full_addr + cur.stage * 8;
            mbar_arrive_expect_tx(bar, TILE);
            tma_load_2d(ring_addr + cur.stage * STAGE_BYTES, kv ? tmv : tmk, h * D, ch * KV_TILE, bar, policy);
            cur.advance();
            ++issued;
        }
    }
};

// ---------------------------------------------------------------- consumer side
struct Consumer {
    const uint8_t* ring;
    uint32_t full_addr, empty_addr;
    Cursor cur;
    AbortCtl ab;
    int warp, lane;
    bool touch_only;
    float* rsum;  // shared memory, NSLOT x GRAN floats: per-slot row sums of a multi-chunk round

    __device__ __forceinline__ const uint8_t* wait_stage() {
        mbar_wait(full_addr + cur.stage * 8, cur.phase, ab, ST_TIMEOUT_FULL);
        return ring + static_cast<size_t>(cur.stage) * STAGE_BYTES;
    }
    __device__ __forceinline__ void release_stage() {
        __syncwarp();
        if (lane == 0) mbar_arrive(empty_addr + cur.stage * 8);
        cur.advance();
    }
    // Mirror of Producer::rows_phase.  xs = activations in shared memory (KC*256
    // floats); epi(granule index relative to g0=0, row in granule, dot product).
    // gate_chunk >= 0: before the first use of activation chunk `gate_chunk`, wait (bounded)
    // on mbarrier gate_bar / gate_parity (the helpers' "chunks from here on are ready").
    template <class Epi>
    __device__ __forceinline__ void rows_phase(int cnt, int KC, const float* xs, Epi epi, int gate_chunk = -1,
                                               uint32_t gate_bar = 0, uint32_t gate_parity = 0) {
        if (cnt <= 0) return;
        const int nr = ceil_div(cnt, NSLOT), base = cnt / nr, extra = cnt % nr;
        int g = 0;
        for (int r = 0; r < nr; ++r) {
            const int n = base + (r < extra ? 1 : 0);
            const bool a0 = warp < n, a1 = warp + NCWARP < n;
            float acc0[GRAN], acc1[GRAN];
#pragma unroll
            for (int i = 0; i < GRAN; ++i) acc0[i] = acc1[i] = 0.f;
            for (int c = 0; c < KC; ++c) {
                // (probed with a pause: eight warps probing an mbarrier back to back take issue slots and
                // shared-memory pipe cycles from the helper warps they are waiting for)
                if (c == gate_chunk && r == 0)
                    wait_bounded<POLL_BACKOFF_NS>([&] { return mbar_try_wait(gate_bar, gate_parity); }, ab, ST_TIMEOUT_FULL);
                const uint8_t* st = wait_stage();
                if (!touch_only) {
                    if (a0) gemv_slot(st + warp * SLOT_BYTES, xs + c * KCHUNK, lane, acc0);
                    if (a1) gemv_slot(st + (warp + NCWARP) * SLOT_BYTES, xs + c * KCHUNK, lane, acc1);
                }
                release_stage();
            }
            if (a0) {
                const float v = warp_reduce8(acc0, lane);
                if ((lane & 3) == 0) epi(g + warp, reduce8_row(lane), v);
            }
            if (a1) {
                const float v = warp_reduce8(acc1, lane);
                if ((lane & 3) == 0) epi(g + warp + NCWARP, reduce8_row(lane), v);
            }
            g += n;
        }
    }
    // Mirror of Producer::rows_phase2.  Granule v < cntA multiplies xsA and reports to epiA(v, row,
    // dot), the others xsB / epiB(v - cntA, ...).  after_a() runs once, by all consumer threads,
    // right after the round that finishes A's last granule (at once when cntA == 0).
    template <class EpiA, class EpiB, class AfterA>
    __device__ __forceinline__ void rows_phase2(int cntA, int cntB, int KC, const float* xsA, const float* xsB, EpiA epiA,
                                                EpiB epiB, AfterA after_a) {
        const int cnt = cntA + cntB;
        bool a_done = false;
        if (cntA == 0) {
            after_a();
            a_done = true;
        }
        if (cnt <= 0) return;
        int np;
        const int m = plan_rounds(cnt, KC, np);
        if (m > 1) {
            // mirror of the producer's multi-chunk stages; the chunk partials of a row meet in rsum
            const int tid = warp * 32 + lane;
            for (int g = 0; g < cnt; g += np) {
                const int n = min(np, cnt - g);
                const int gi0 = warp % n, cc0 = warp / n, gi1 = (warp + NCWARP) % n, cc1 = (warp + NCWARP) / n;
                const float* x0 = (g + gi0 < cntA) ? xsA : xsB;
                const float* x1 = (g + gi1 < cntA) ? xsA : xsB;
                float acc0[GRAN], acc1[GRAN];
#pragma unroll
                for (int i = 0; i < GRAN; ++i) acc0[i] = acc1[i] = 0.f;
                for (int c0 = 0; c0 < KC; c0 += m) {
                    const int mt = min(m, KC - c0);
                    const uint8_t* st = wait_stage();
                    if (!touch_only) {
                        if (warp < n * mt) gemv_slot(st + warp * SLOT_BYTES, x0 + (c0 + cc0) * KCHUNK, lane, acc0);
                        if (warp + NCWARP < n * mt) gemv_slot(st + (warp + NCWARP) * SLOT_BYTES, x1 + (c0 + cc1) * KCHUNK, lane, acc1);
                    }
                    release_stage();
                }
                if (warp < n * m) {
                    const float v = warp_reduce8(acc0, lane);
                    if ((lane & 3) == 0) rsum[warp * GRAN + reduce8_row(lane)] = v;
                }
                if (warp + NCWARP < n * m) {
                    const float v = warp_reduce8(acc1, lane);
                    if ((lane & 3) == 0) rsum[(warp + NCWARP) * GRAN + reduce8_row(lane)] = v;
                }
                consumer_sync(NCTHR);
                if (tid < n * GRAN) {
                    const int gi = tid / GRAN, r = tid - gi * GRAN;
                    float v = 0.f;
                    for (int cc = 0; cc < m; ++cc) v += rsum[(cc * n + gi) * GRAN + r];  // chunk order: fixed
                    if (g + gi < cntA) epiA(g + gi, r, v);
                    else epiB(g + gi - cntA, r, v);
                }
                consumer_sync(NCTHR);  // rsum is rewritten by the next round
                if (!a_done && g + n >= cntA) {
                    after_a();
                    a_done = true;
                }
            }
            return;
        }
        const int nr = ceil_div(cnt, NSLOT), base = cnt / nr, extra = cnt % nr;
        int g = 0;
        for (int r = 0; r < nr; ++r) {
            const int n = base + (r < extra ? 1 : 0);
            const int v0 = g + warp, v1 = g + warp + NCWARP;
            const bool a0 = warp < n, a1 = warp + NCWARP < n;
            const float* x0 = (v0 < cntA) ? xsA : xsB;
            const float* x1 = (v1 < cntA) ? xsA : xsB;
            float acc0[GRAN], acc1[GRAN];
#pragma unroll
            for (int i = 0; i < GRAN; ++i) acc0[i] = acc1[i] = 0.f;
            for (int c = 0; c < KC; ++c) {
                const uint8_t* st = wait_stage();
                if (!touch_only) {
                    if (a0) gemv_slot(st + warp * SLOT_BYTES, x0 + c * KCHUNK, lane, acc0);
                    if (a1) gemv_slot(st + (warp + NCWARP) * SLOT_BYTES, x1 + c * KCHUNK, lane, acc1);
                }
                release_stage();
            }
            if (a0) {
                const float v = warp_reduce8(acc0, lane);
                if ((lane & 3) == 0) {
                    if (v0 < cntA) epiA(v0, reduce8_row(lane), v);
                    else epiB(v0 - cntA, reduce8_row(lane), v);
                }
            }
            if (a1) {
                const float v = warp_reduce8(acc1, lane);
                if ((lane & 3) == 0) {
                    if (v1 < cntA) epiA(v1, reduce8_row(lane), v);
                    else epiB(v1 - cntA, reduce8_row(lane), v);
                }
            }
            g += n;
            if (!a_done && g >= cntA) {
                after_a();
                a_done = true;
            }
        }
    }
};

// ---------------------------------------------------------------- the kernel
// P3's attention chunks of xbuf = weighted sums of the partial records (record offsets in offs[], normalised
// weights in pm[], both complete when this runs).  Run by threads t = 0 .. nthr-1 whose named barrier is bar_id:
// four consecutive elements per thread, two groups of eight records in flight.  mseg > 1: a vector's records are
// cut into mseg segments that different threads sum, so that every thread has loads in flight; the segment sums
// meet in the (idle) auxiliary region of xbuf and are added in segment order.  Run by the helper warps.  (Run by
// the 256 consumer threads instead, which are idle by then on a tensor-parallel shard, it passed its tests but cost
// more than it saved: as a real function call 7 % per token -- every live register of the streaming loops is saved
// around the call -- and inlined into the consumers' code it spilled 170 bytes per thread.)
struct MergeArgs {
    float* xbuf;
    const int* offs;
    const float* pm;
    const float* pbase;
    int aux_off, nve, mseg, pstr, nmid, me, KVW;
};
template <int D, int CS>
__device__ __forceinline__ void merge_sums(const MergeArgs& a, int t, int nthr, int bar_id) {
    constexpr int HPC = heads_per_chunk(D);
    const int nve = a.nve, mseg = a.mseg, pstr = a.pstr;
    const int seglen = ceil_div(ceil_div(pstr, mseg), 8) * 8;
    float4* segbuf = reinterpret_cast<float4*>(a.xbuf + a.aux_off);
    const int nitem = nve * mseg;
    for (int v0 = t; v0 < nitem; v0 += 2 * nthr) {
        float4 acc[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
        int wrow[2], dd[2], dsti[2], jlo[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
            const int item = v0 + u * nthr;
            const int sg = item / nve, v = item - sg * nve;
            const int i = v / (KCHUNK / 4), k4 = v - i * (KCHUNK / 4);
            const int q = a.me + i * CS;
            const int e = q * KCHUNK + k4 * 4;
            wrow[u] = -1;
            dd[u] = 0;
            jlo[u] = sg * seglen;
            dsti[u] = (item < nitem) ? (mseg > 1 ? item : (a.nmid + i) * KCHUNK + k4 * 4) : -1;
            if (item < nitem && e < a.KVW) {
                const int h = e / D;
                dd[u] = e - h * D;
                wrow[u] = (i * HPC + (h - (q * KCHUNK) / D)) * pstr;
            }
        }
        for (int j0 = 0; j0 < seglen; j0 += 8) {
            float4 vv[2][8];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    vv[u][jj] = make_float4(0.f, 0.f, 0.f, 0.f);
                    const int j = jlo[u] + j0 + jj;
                    if (wrow[u] >= 0 && j < pstr) {
                        const int o = a.offs[wrow[u] + j];
                        if (o >= 0) vv[u][jj] = ld_cg_f32x4(a.pbase + o + dd[u]);
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int jj = 0; jj < 8; ++jj) {
                    const int j = jlo[u] + j0 + jj;
                    const float w = (wrow[u] >= 0 && j < pstr) ? a.pm[wrow[u] + j] : 0.f;
                    acc[u].x = fmaf(w, vv[u][jj].x, acc[u].x);
                    acc[u].y = fmaf(w, vv[u][jj].y, acc[u].y);
                    acc[u].z = fmaf(w, vv[u][jj].z, acc[u].z);
                    acc[u].w = fmaf(w, vv[u][jj].w, acc[u].w);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 2; ++u)
            if (dsti[u] >= 0) {
                if (mseg > 1) segbuf[dsti[u]] = acc[u];
                else *reinterpret_cast<float4*>(a.xbuf + dsti[u]) = acc[u];
            }
    }
    if (mseg > 1) {
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthr) : "memory");
        for (int v = t; v < nve; v += nthr) {
            float4 r = segbuf[v];
            for (int sg = 1; sg < mseg; ++sg) {
                const float4 o = segbuf[sg * nve + v];
                r.x += o.x;
                r.y += o.y;
                r.z += o.z;
                r.w += o.w;
            }
            const int i = v / (KCHUNK / 4), k4 = v - i * (KCHUNK / 4);
            *reinterpret_cast<float4*>(a.xbuf + (a.nmid + i) * KCHUNK + k4 * 4) = r;
        }
        // the sums are in place for every thread; the auxiliary region may be rewritten
        asm volatile("bar.sync %0, %1;" ::"r"(bar_id), "r"(nthr) : "memory");
    }
}

// The whole launch of one parameter block: every thread of the CTA calls it.  `kv_maps` is the address of
// Params::kv_maps in memory the TMA unit can read a tensor map from (kernel parameters or global memory -- not the
// shared-memory copy of the parameters that a multi-block launch works from).
template <int D, int CS>
__device__ __forceinline__ void decode_body(const Params& p, const CUtensorMap* kv_maps, uint8_t* smem_raw) {
    static_assert(D % 8 == 0 && D <= 128, "head_dim must be a multiple of 8, at most 128");
    // one attention partial: D numerators, running max, denominator, padded so that every
    // record (and every 4-element group in it) starts on a 16-byte boundary
    constexpr int PREC = D + 4;
    const Smem sm = carve(smem_raw, p.nstage, p.xbuf_floats);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int G = gridDim.x, cta = blockIdx.x;
    const AbortCtl ab{sm.abort_flag, p.status};

    if (tid == 0) {
        *sm.abort_flag = 0;
        for (int s = 0; s < p.nstage; ++s) {
            mbar_init(smem_u32(sm.full + s), 1);
            mbar_init(smem_u32(sm.empty + s), NCWARP);
        }
        mbar_init(smem_u32(sm.xbar), NCWARP * CS);
        mbar_init(smem_u32(sm.h_go), 1);
        mbar_init(smem_u32(sm.attn_ready), NHWARP);
        mbar_init(smem_u32(sm.mid_ready), 1);
        mbar_init(smem_u32(sm.h_layer), 1);
        for (int i = 0; i < MAXHPC; ++i) mbar_init(smem_u32(sm.q_ready + i), NHWARP);
        mbar_init(smem_u32(sm.pf_ready), NCWARP);
        mbar_init(smem_u32(sm.pf_free), NFWARP);
        mbar_fence_init();
    }
    __syncthreads();
    if constexpr (CS > 1) dsm::cluster_sync_all();  // peers' barriers exist before any remote arrive
    // the launch after this one may take an SM as soon as a CTA of this grid leaves it
    if (p.pdl && tid == 0) griddep_launch_dependents();

    const int seq = p.seq_ptr ? __ldcg(p.seq_ptr) : p.seq_host;
    const int H = p.H, NH = p.NH, R = p.R, F = p.F;
    const int KVW = NH * D;  // cache row width held by this rank
    {
        // all CTAs see the same seq, so they all leave together
        int kv_rows_min = 0x7fffffff;
        if (p.phase_mask & PH_P2)
            for (int l = 0; l < p.n_layers; ++l) kv_rows_min = min(kv_rows_min, p.kv_inline ? p.kv_rows_inline : p.layers[l].kv_rows);
        const int spare = (p.arch_flags & AF_NO_APPEND) ? 0 : 1;  // a free row for the new token
        if (seq < 0 || ((p.phase_mask & PH_P2) && seq > kv_rows_min - spare)) {
            if (tid == 0) atomicCAS(p.status, 0, ST_BAD_SEQ);
            return;
        }
    }

    // ---- static work split (identical on producer and consumer side)
    const int KC1 = ceil_div(H, KCHUNK);
    const int NGq = (p.arch_flags & AF_NO_QKV) ? 0 : (3 * KVW) / GRAN;
    const int NGu = (p.F_up ? p.F_up : F) / GRAN, NG1 = NGq + NGu;
    // Every CTA streams a share of the QKV rows first and a share of the MLP-up rows after it, as
    // one sequence of granules.  The up share is cut so that QKV + up together are as even as the
    // grid allows (p1_joint, verified by the host); otherwise each is split evenly on its own.
    int qa = 0, qb = 0, ua = 0, ub = 0;  // QKV granules [qa, qb), up granules [ua, ub)
    if (p.p1_joint >= 2) {
        // grouped: CTAs [0, Gq) share the QKV rows, CTAs [Gq, G) the MLP-up rows
        int Gq = (NGu == 0) ? G : (NGq == 0 ? 0 : p.gq);
        if (NGq > 0 && NGu > 0) Gq = max(1, min(G - 1, Gq));
        const int vc = (p.p1_joint == 3) ? G - 1 - cta : cta;
        if (vc < Gq) {
            qa = part_begin(vc, NGq, Gq);
            qb = part_begin(vc + 1, NGq, Gq);
        } else {
            ua = part_begin(vc - Gq, NGu, G - Gq);
            ub = part_begin(vc - Gq + 1, NGu, G - Gq);
        }
    } else {
        qa = part_begin(cta, NGq, G);
        qb = part_begin(cta + 1, NGq, G);
        if (p.p1_joint == 1) {
            ua = part_begin(cta, NG1, G) - qa;
            ub = part_begin(cta + 1, NG1, G) - qb;
        } else {
            ua = part_begin(cta, NGu, G);
            ub = part_begin(cta + 1, NGu, G);
        }
    }
    const int nch = ceil_div(seq, KV_TILE);
    const int T2 = NH * nch;
    const int t2a = part_begin(cta, T2, G), t2b = part_begin(cta + 1, T2, G);
    const int NC = G / CS, cl = cta / CS;
    const int me = (CS > 1) ? static_cast<int>(dsm::cta_rank()) : 0;
    const int NG3 = H / GRAN;
    const int g3a = part_begin(cl, NG3, NC), g3b = part_begin(cl + 1, NG3, NC);
    const int KCo = (p.p3_flags & F3_USE_O) ? ceil_div(KVW, KCHUNK) : 0;
    const int KCd = (p.p3_flags & F3_USE_DOWN) ? ceil_div(F, KCHUNK) : 0;
    const int KC3 = KCo + KCd;
    const int my3 = (KC3 > me) ? ceil_div(KC3 - me, CS) : 0;  // chunks me, me+CS, ...
    // attention merge tables (P3): my chunks that hold attention, heads touching a
    // chunk, partial slots per head
    constexpr int HPC = heads_per_chunk(D);
    const int nattn = (KCo > me) ? ceil_div(KCo - me, CS) : 0;
    const int pstr = (nch == 0) ? 1 : min(MAX_PARTS, ceil_div(G, NH) + 2);
    int NG4 = 0, g4a = 0, g4b = 0;
    if (p.phase_mask & PH_P4) {
        NG4 = ceil_div(p.tail->vocab, GRAN);
        g4a = part_begin(cta, NG4, G);
        g4b = part_begin(cta + 1, NG4, G);
    }

    // This CTA's MLP chunks of P3's activation vector, fp32 in xbuf, chunk-major from offset 0: copied
    // (or, for SwiGLU, formed as silu(gate) * up) from the fp32 intermediate that P1 left in global
    // memory.  Called by `nthr` threads with t = 0 .. nthr-1; copies are asynchronous (the caller
    // waits with cp.async.wait_all).
    auto stage_mid = [&](int t, int nthr) {
        const int nmid_ = my3 - nattn;
        const int nvec = nmid_ * (KCHUNK / 4);
        if (p.arch_flags & AF_SWIGLU) {
            // mid[e] = silu(gate[e]) * up[e], gate rows at [0, F), up rows at [F, 2F) of the scratch
            for (int v0 = t; v0 < nvec; v0 += nthr * 4) {
                float4 gv[4], uv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * nthr;
                    gv[u] = uv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (v < nvec) {
                        const int i = v / (KCHUNK / 4), k4 = v % (KCHUNK / 4);
                        const int e = (me + (nattn + i) * CS - KCo) * KCHUNK + k4 * 4;  // F is a multiple of 8
                        if (e < F) {
                            gv[u] = ld_cg_f32x4(p.mid_f32 + e);
                            uv[u] = ld_cg_f32x4(p.mid_f32 + F + e);
                        }
                    }
                }
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const int v = v0 + u * nthr;
                    if (v < nvec) {
                        const int i = v / (KCHUNK / 4), k4 = v % (KCHUNK / 4);
                        float4 o;
                        o.x = gv[u].x / (1.f + __expf(-gv[u].x)) * uv[u].x;
                        o.y = gv[u].y / (1.f + __expf(-gv[u].y)) * uv[u].y;
                        o.z = gv[u].z / (1.f + __expf(-gv[u].z)) * uv[u].z;
                        o.w = gv[u].w / (1.f + __expf(-gv[u].w)) * uv[u].w;
                        *reinterpret_cast<float4*>(sm.xbuf + i * KCHUNK + k4 * 4) = o;
                    }
                }
            }
        } else {
            // asynchronous 16-byte copies of the fp32 intermediate straight into xbuf
            for (int v = t; v < nvec; v += nthr) {
                const int i = v / (KCHUNK / 4), k4 = v % (KCHUNK / 4);
                const int e = (me + (nattn + i) * CS - KCo) * KCHUNK + k4 * 4;
                float* dst = sm.xbuf + i * KCHUNK + k4 * 4;
                if (e + 3 < F) {
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)),
                                 "l"(p.mid_f32 + e) : "memory");
                } else {
                    for (int k = 0; k < 4; ++k) dst[k] = (e + k < F) ? ld_cg_f32(p.mid_f32 + e + k) : 0.f;
                }
            }
            asm volatile("cp.async.commit_group;" ::: "memory");
        }
    };

    // =========================================================== producer warp
    if (warp == NCWARP) {
        if (lane == 0) {
            Producer pr;
            pr.ring_addr = smem_u32(sm.ring);
            pr.full_addr = smem_u32(sm.full);
            pr.empty_addr = smem_u32(sm.empty);
            pr.cur = Cursor{0, 0u, p.nstage};
            pr.policy = l2_policy_evict_first();
            pr.ab = ab;
            pr.issued = 0;
            // the first ring-full of weight stages does not depend on the kernel before this one
            pr.early_left = (p.pdl && (p.phase_mask & PH_P1)) ? p.nstage : -1;
            if (p.pdl && pr.early_left < 0) griddep_wait();

            for (int l = 0; l < p.n_layers; ++l) {
                const LayerDesc* L = p.layers + l;
                if (p.phase_mask & PH_P1) {
                    pr.rows_phase2(&L->tm_qkv, qa, qb - qa, &L->tm_up, ua, ub - ua, KC1);
                    trace_mark(p, cta, l, TR_PROD_P1);
                }
                pr.depend();  // key / value tiles and everything after them may come from the preceding kernel
                if (p.phase_mask & PH_P2) {
                    const CUtensorMap* tmk = p.kv_inline ? kv_maps : &L->tm_k;
                    const CUtensorMap* tmv = p.kv_inline ? kv_maps + 1 : &L->tm_v;
                    for (int t = t2a; t < t2b; ++t) pr.kv_stage<D>(tmk, tmv, t / nch, t % nch);
                    trace_mark(p, cta, l, TR_PROD_P2);
                }
                if (p.phase_mask & PH_P3) {
                    const int cnt = g3b - g3a;
                    if (cnt > 0 && my3 > 0) {
                        const int nr = ceil_div(cnt, NSLOT), base = cnt / nr, extra = cnt % nr;
                        int g = g3a;
                        for (int r = 0; r < nr; ++r) {
                            const int n = base + (r < extra ? 1 : 0);
                            // MLP chunks first: the attention chunks are merged by the helper
                            // warps while these stream
                            for (int i = nattn; i < my3; ++i)
                                pr.rows_stage(&L->tm_down, (me + i * CS - KCo) * KCHUNK, g, n);
                            for (int i = 0; i < nattn; ++i) pr.rows_stage(&L->tm_o, (me + i * CS) * KCHUNK, g, n);
                            g += n;
                        }
                    }
                    trace_mark(p, cta, l, TR_PROD_P3);
                }
            }
            // (the LM head as the second matrix of a two-matrix phase whose first matrix is empty)
            if (p.phase_mask & PH_P4) pr.rows_phase2(&p.tail->tm_head, 0, 0, &p.tail->tm_head, g4a, g4b - g4a, KC1);
            // After an abort the consumers stop draining the ring: give the copies
            // already issued a bounded chance to land before this CTA's shared
            // memory goes away.
            if (*ab.flag) {
                const unsigned long long t0 = globaltimer_ns();
                const uint32_t back = min(pr.issued, static_cast<uint32_t>(p.nstage));
                Cursor c = pr.cur;
                for (uint32_t k = 0; k < back; ++k) {
                    // step the cursor back one stage
                    if (c.stage == 0) { c.stage = c.nstage - 1; c.phase ^= 1u; } else { --c.stage; }
                    const uint32_t bar = pr.full_addr + c.stage * 8;
                    while (!mbar_try_wait(bar, c.phase)) {
                        if (globaltimer_ns() - t0 > WAIT_LIMIT_NS) {
                            atomicCAS(p.status, ST_OK, ST_TIMEOUT_DRAIN);
                            break;
                        }
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp > NCWARP) {
        // ========================================================= helper warps
        if (p.pdl) griddep_wait();
        // Side work that is pure L2 latency, kept off the consumers' path: in P3, merge the
        // attention partials of all CTAs into this CTA's attention chunks of xbuf.
        const int ht = tid - (NCWARP + 1) * 32;
        const int nent = nattn * HPC * pstr;
        // P3's attention merge (merge_sums above): with many partials per head (few local heads, i.e. tensor parallel)
        // a vector's records are cut into mseg segments.
        MergeArgs mga;
        mga.xbuf = sm.xbuf;
        mga.offs = sm.offs;
        mga.pm = sm.pm;
        mga.pbase = (nch == 0) ? p.attn_new : p.attn_part;
        mga.aux_off = p.aux_off;
        mga.nve = nattn * (KCHUNK / 4);
        mga.mseg = (mga.nve > 0) ? max(1, min(ceil_div(pstr, 8), (aux_floats(D) / 4) / mga.nve)) : 1;
        if (p.merge_seg_max > 0) mga.mseg = min(mga.mseg, p.merge_seg_max);
        mga.pstr = pstr;
        mga.nmid = my3 - nattn;
        mga.me = me;
        mga.KVW = KVW;
        const float* pbase = mga.pbase;

        // every CTA past P1 <=> the MLP intermediate is complete: one helper thread watches the
        // count and tells the consumers through shared memory, so that they never poll global memory
        const bool mid_wait = (p.phase_mask & PH_P1) && (p.phase_mask & PH_P3) && !(p.p3_flags & F3_MID_F16);
        // Helper warp 0: one thread watches the count, then the warp copies this CTA's MLP chunks into
        // xbuf -- the consumers are in P2 meanwhile (xbuf's chunk area is free once every CTA, this one
        // included, is past P1) and find their P3 operands in place when they arrive.  In a launch without
        // P2 the consumers would only wait for that one warp: there it just passes the signal on and the
        // consumer threads stage the chunks themselves.
        const bool mid_by_helper = mid_wait && (p.phase_mask & PH_P2);
        auto watch_mid = [&](int l) {
            if (mid_wait && ht < 32) {
                if (ht == 0) {
                    const unsigned target = static_cast<unsigned>(l + 1) * static_cast<unsigned>(G);
                    wait_bounded<POLL_BACKOFF_NS>([&] { return ld_acquire_u32(p.sync + 3) >= target; }, ab, ST_TIMEOUT_GRID);
                    __threadfence();
                }
                __syncwarp();
                if (mid_by_helper) {
                    stage_mid(ht, 32);
                    asm volatile("cp.async.wait_all;" ::: "memory");
                    __syncwarp();
                }
                if (ht == 0) mbar_arrive(smem_u32(sm.mid_ready));
            }
        };
        const bool do_merge = (p.phase_mask & PH_P3) && nattn > 0;
        // P2 set-up done ahead of the consumers: the rotated, scaled query of every head this CTA
        // streams, and the new token's key and value where it streams the head's last chunk
        // (appended to the cache here), as fp32 in the spare region of xbuf.  The q/k/v words are
        // polled while the consumers are still in P1.
        const bool do_q = (p.phase_mask & PH_P2) && nch > 0 && t2b > t2a;
        const unsigned hl_base = __ldcg(p.epoch_base);
        uint32_t lpar = 0;
        auto stage_q = [&](int l) {
            mbar_wait(smem_u32(sm.h_layer), lpar, ab, ST_TIMEOUT_GRID);
            lpar ^= 1u;
            const LayerDesc* L = p.layers + l;
            const QkvView qkv{p.qkv_ll, hl_base + static_cast<unsigned>(l) + 1u, p.qkv_any_epoch != 0, &ab};
            const int pos_off = p.rope_stride * seq;
            const float* cosr = p.cos + pos_off;
            const float* sinr = p.sin + pos_off;
            const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(D));
            float* qpre = sm.xbuf + p.aux_off;
            const int h_first = t2a / nch, h_last = (t2b - 1) / nch;
            const int half_r = R >> 1;
            // elements [e_lo, e_hi) of head h's [q; k; v] vector: rotate, scale / round, leave in xbuf
            // (and, for k and v, in the cache row and the k_new / v_new outputs)
            auto stage_range = [&](int h, int e_lo, int e_hi) {
                const int qi = h * 3 * D;
                float* dst = qpre + (h - h_first) * 3 * D;
                // all of this thread's words (and their rotation partners) in flight at once; the
                // epochs are checked together and the batch is re-read (bounded) until all match
                constexpr int KQ = (2 * D + NHTHR - 1) / NHTHR;
                uint2 w[KQ], wp[KQ];
                auto fetch = [&]() {
                    bool ok = true;
#pragma unroll
                    for (int k = 0; k < KQ; ++k) {
                        const int e = e_lo + ht + k * NHTHR;
                        if (e < e_hi) {
                            const int part = e / D, d = e - part * D;
                            w[k] = ld_ll(qkv.base + qi + e);
                            ok = ok && (qkv.any || w[k].y == qkv.epoch);
                            if (part < 2 && d < R) {
                                wp[k] = ld_ll(qkv.base + qi + e + (d < half_r ? half_r : -half_r));
                                ok = ok && (qkv.any || wp[k].y == qkv.epoch);
                            }
                        }
                    }
                    return ok;
                };
                if (!fetch()) wait_bounded<POLL_BACKOFF_NS>(fetch, ab, ST_TIMEOUT_PEER);
#pragma unroll
                for (int k = 0; k < KQ; ++k) {
                    const int e = e_lo + ht + k * NHTHR;
                    if (e >= e_hi) continue;
                    const int part = e / D, d = e - part * D;
                    float val = __uint_as_float(w[k].x);
                    if (part < 2 && d < R) {
                        const float partner = __uint_as_float(wp[k].x);
                        val = val * __ldg(cosr + d) + ((d < half_r) ? -partner : partner) * __ldg(sinr + d);
                    }
                    if (part == 0) {
                        dst[d] = val * qscale;
                    } else {
                        const __half h16 = __float2half_rn(val);
                        dst[part * D + d] = __half2float(h16);
                        const size_t off = static_cast<size_t>(seq) * KVW + h * D + d;
                        if (part == 1) {
                            if (!(p.arch_flags & AF_NO_APPEND)) L->k_cache[off] = h16;
                            if (p.k_new) p.k_new[h * D + d] = h16;
                        } else {
                            if (!(p.arch_flags & AF_NO_APPEND)) L->v_cache[off] = h16;
                            if (p.v_new) p.v_new[h * D + d] = h16;
                        }
                    }
                }
            };
            // the queries first, head by head, each released to the consumers as soon as it is there ...
            for (int h = h_first; h <= h_last; ++h) {
                stage_range(h, 0, D);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(sm.q_ready + (h - h_first)));
            }
            // ... then the new token's key and value where this CTA streams the head's last chunk: only the
            // helper warps that finish the partials need them
            for (int h = h_first; h <= h_last; ++h)
                if ((h + 1) * nch - 1 < t2b) stage_range(h, D, 3 * D);
            helper_sync(NHTHR);
        };
        {
            // Which partial feeds which of my chunks depends only on (grid, seq): tabulate once.
            for (int it = ht; do_merge && it < nent; it += NHTHR) {
                const int pair = it / pstr, j = it - pair * pstr;
                const int i = pair / HPC, hh = pair - i * HPC;
                const int q = me + i * CS;
                const int h = (q * KCHUNK) / D + hh;
                int off = -1;
                if (h < NH && h * D < min((q + 1) * KCHUNK, KVW)) {
                    if (nch == 0) {
                        if (j == 0) off = h * PREC;
                    } else {
                        const int c = part_of(h * nch, T2, G) + j;
                        if (c <= part_of((h + 1) * nch - 1, T2, G)) {
                            const int b0 = part_begin(c, T2, G);
                            // CTAs between the first and last may own no item at all (T2 < G)
                            if (part_begin(c + 1, T2, G) != b0) off = (c * MAXL + (h - b0 / nch)) * PREC;
                        }
                    }
                }
                sm.offs[it] = off;
            }
            helper_sync(NHTHR);
            constexpr int ML_ITERS = (WTS_SLOTS + NHTHR - 1) / NHTHR;
            uint32_t gpar = 0;
            unsigned nfin = 0;  // partials finished so far (all layers): phase of the hand-over barriers
            // Helper warps 1..NFWARP finish this CTA's attention partials.  The consumers leave a head's
            // per-warp running state (numerators, max, denominator) in the hand-over buffer and go on
            // with the next head or with P3; here the NCWARP slots are combined in a fixed order, the
            // token being decoded is folded in where this CTA streamed the head's last chunk (its
            // rotated key and value are still in the pre-staged region), and the record is written and
            // stamped for the CTAs that merge it.
            auto finish_partials = [&](int l) {
                const int ft = ht - 32;  // 0 .. NFTHR-1
                const int h_first = t2a / nch, h_last = (t2b - 1) / nch;
                const float* qpre = sm.xbuf + p.aux_off;
                const float* hb = qpre + MAXHPC * 3 * D;   // [NCWARP][D]
                const float* hml = hb + NCWARP * D;        // [NCWARP][2]
                const unsigned pep = hl_base + static_cast<unsigned>(l) + 1u;
                for (int h = h_first; h <= h_last; ++h) {
                    const bool has_last = (h + 1) * nch - 1 < t2b;
                    const float* hq = qpre + (h - h_first) * 3 * D;
                    mbar_wait(smem_u32(sm.pf_ready), nfin & 1u, ab, ST_TIMEOUT_GRID);
                    float s_new = -INFINITY;
                    if (has_last) {
                        // score of the new token: q (already scaled) . k_new, summed in a fixed order
                        float part = 0.f;
                        for (int d = ft; d < D; d += NFTHR) part = fmaf(hq[d], hq[D + d], part);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
                        if (lane == 0) sm.red[40 + (ft >> 5)] = part;
                        fin_sync();
                        s_new = 0.f;
#pragma unroll
                        for (int i = 0; i < NFWARP; ++i) s_new += sm.red[40 + i];
                    }
                    float M = s_new;
#pragma unroll
                    for (int i = 0; i < NCWARP; ++i) M = fmaxf(M, hml[i * 2]);
                    float wgt[NCWARP], lsum = 0.f;
#pragma unroll
                    for (int i = 0; i < NCWARP; ++i) {
                        const float mi = hml[i * 2];
                        wgt[i] = (mi > -INFINITY) ? exp2f(mi - M) : 0.f;
                        lsum = fmaf(hml[i * 2 + 1], wgt[i], lsum);
                    }
                    const float wn = has_last ? exp2f(s_new - M) : 0.f;
                    lsum += wn;
                    float* dst = p.attn_part + (static_cast<size_t>(cta) * MAXL + (h - h_first)) * PREC;
                    for (int d = ft; d < D; d += NFTHR) {
                        float a = 0.f;
#pragma unroll
                        for (int i = 0; i < NCWARP; ++i) a = fmaf(hb[i * D + d], wgt[i], a);
                        if (has_last) a = fmaf(wn, hq[2 * D + d], a);
                        dst[d] = a;
                    }
                    if (ft == 0) {
                        dst[D] = M;
                        dst[D + 1] = lsum;
                    }
                    fin_sync();  // record written, hand-over buffer read by everybody
                    if (ft == 0) publish_record(dst + D + 2, pep);
                    if (lane == 0) mbar_arrive(smem_u32(sm.pf_free));
                    ++nfin;
                }
            };
            for (int l = 0; l < p.n_layers; ++l) {
                if (do_q) stage_q(l);
                if (do_q && ht >= 32 && ht < 32 + NFTHR) finish_partials(l);
                if (p.phase_mask & PH_P3) watch_mid(l);
                if (!do_merge) {
                    if (do_q) helper_sync(NHTHR);  // the pre-staged region is rewritten only after its last reader
                    continue;
                }
                // the consumers have left P2 of this layer: xbuf's attention chunks are free
                mbar_wait(smem_u32(sm.h_go), gpar, ab, ST_TIMEOUT_GRID);
                gpar ^= 1u;
                if (ht == 0) trace_mark(p, cta, l, TR_MERGE_GO);
                const unsigned pep = hl_base + static_cast<unsigned>(l) + 1u;
                // (max, denominator) of every table entry -> normalised weights in pm[]
                float mreg[ML_ITERS], lreg[ML_ITERS];
#pragma unroll
                for (int k = 0; k < ML_ITERS; ++k) {
                    const int it = ht + k * NHTHR;
                    mreg[k] = -INFINITY;
                    lreg[k] = 0.f;
                    if (it < nent) {
                        const int o = sm.offs[it];
                        if (o >= 0) {
                            // no grid barrier after P2: every record carries the epoch of its layer,
                            // stamped after its contents; poll it (bounded) before reading the record
                            if (!p.part_any_epoch) {
                                const unsigned* ew = reinterpret_cast<const unsigned*>(pbase + o + D + 2);
                                if (ld_acquire_u32(ew) != pep)
                                    wait_bounded<POLL_BACKOFF_NS>([&] { return ld_acquire_u32(ew) == pep; }, ab, ST_TIMEOUT_GRID);
                            }
                            mreg[k] = ld_cg_f32(pbase + o + D);
                            lreg[k] = ld_cg_f32(pbase + o + D + 1);
                        }
                    }
                }
#pragma unroll
                for (int k = 0; k < ML_ITERS; ++k) {
                    const int it = ht + k * NHTHR;
                    if (it < nent) {
                        sm.pm[it] = mreg[k];
                        sm.pl[it] = lreg[k];
                    }
                }
                helper_sync(NHTHR);
                if (ht == 0) trace_mark(p, cta, l, TR_MERGE_POLLED);
                // normalised weights, one helper warp per (chunk, head) row of the table: lane j holds slots j and
                // j + 32 (a head has at most MAX_PARTS = 64 partials); maximum and denominator by butterfly
                // shuffles -- a fixed order, the same in every CTA and on every rank
                static_assert(MAX_PARTS <= 64, "two slots per lane");
                {
                    const int hw = ht >> 5;
                    const int nrow = nattn * HPC;
                    for (int r = hw; r < nrow; r += NHWARP) {
                        const int r0 = r * pstr;
                        const bool a0 = lane < pstr, a1 = lane + 32 < pstr;
                        const float m0 = a0 ? sm.pm[r0 + lane] : -INFINITY, m1 = a1 ? sm.pm[r0 + lane + 32] : -INFINITY;
                        const float l0 = a0 ? sm.pl[r0 + lane] : 0.f, l1 = a1 ? sm.pl[r0 + lane + 32] : 0.f;
                        float M = fmaxf(m0, m1);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
                        const float e0 = (m0 > -INFINITY) ? exp2f(m0 - M) : 0.f, e1 = (m1 > -INFINITY) ? exp2f(m1 - M) : 0.f;
                        float den = fmaf(e0, l0, e1 * l1);
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
                        __syncwarp();  // every lane has read its m before the slots become weights
                        if (a0) sm.pm[r0 + lane] = (e0 > 0.f) ? e0 / den : 0.f;
                        if (a1) sm.pm[r0 + lane + 32] = (e1 > 0.f) ? e1 / den : 0.f;
                    }
                }
                helper_sync(NHTHR);
                merge_sums<D, CS>(mga, ht, NHTHR, 2);
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(sm.attn_ready));
                if (ht == 0) trace_mark(p, cta, l, TR_MERGE_DONE);
            }
        }
    } else {
        // ======================================================= consumer warps
        if (p.pdl) griddep_wait();
        Consumer co;
        co.ring = sm.ring;
        co.full_addr = smem_u32(sm.full);
        co.empty_addr = smem_u32(sm.empty);
        co.cur = Cursor{0, 0u, p.nstage};
        co.ab = ab;
        co.warp = warp;
        co.lane = lane;
        co.touch_only = p.touch_only != 0;
        co.rsum = sm.rsum;
        unsigned epoch = 0;
        uint32_t xparity = 0, hparity = 0, mparity = 0, qpar0 = 0, qpar1 = 0;
        unsigned nflush = 0;  // attention partials handed to the helper warps so far (all layers)
        const bool do_q = (p.phase_mask & PH_P2) && nch > 0 && t2b > t2a;
        const bool mid_wait = (p.phase_mask & PH_P1) && (p.phase_mask & PH_P3) && !(p.p3_flags & F3_MID_F16);
        const int pos_off = p.rope_stride * seq;
        const float* cosr = p.cos + pos_off;
        const float* sinr = p.sin + pos_off;
        const float qscale = 1.4426950408889634f * rsqrtf(static_cast<float>(D));
        // epochs of this launch's flag-in-data handoffs: running base + layer + 1.  The base is a word the
        // last CTA of every launch advances by (layers + 2), so epochs are unique and increasing over
        // launches of any layer count that share the scratch; a zero-filled word never matches
        const unsigned ll_base = __ldcg(p.epoch_base);
        bool need_barrier = false;  // a phase of this launch wrote data the next one reads
        // epochs of this launch's exchanges with the peers, same scheme on a word of their own (all ranks
        // run the same launches, so their words agree)
        const unsigned tp_base = (p.tp_size > 1) ? __ldcg(p.tp_epoch_base) : 0u;

        const __half* x_first = p.embed ? (p.embed + static_cast<size_t>(__ldcg(p.token_in)) * H) : p.x_in;

        for (int l = 0; l < p.n_layers; ++l) {
            const LayerDesc* L = p.layers + l;
            // layer input: the launch's input (plain fp16) or the previous layer's epoch-tagged words
            const __half* x = (l == 0) ? x_first : nullptr;
            const uint2* xll = (l == 0) ? nullptr : p.hid_ll[(l - 1) & 1];
            const unsigned xep = ll_base + static_cast<unsigned>(l);  // = epoch of layer l - 1
            // layer output: plain fp16 for the last layer of the launch, tagged words otherwise
            __half* y = (l == p.n_layers - 1) ? p.out : nullptr;
            uint2* yll = p.hid_ll[l & 1];
            const unsigned yep = ll_base + static_cast<unsigned>(l) + 1u;
            auto store_y = [&](int row, float v) {
                const __half hv = __float2half_rn(v);
                if (y) y[row] = hv;
                else st_ll(yll + row, static_cast<unsigned>(__half_as_ushort(hv)), yep);
            };

            // every consumer thread is past the previous layer's last read of xbuf
            if (do_q && tid == 0) mbar_arrive(smem_u32(sm.h_layer));

            // ------------------------------------------------------------ P1
            if (p.phase_mask & PH_P1) {
                // no grid barrier between layers: the tagged input words are polled by the LayerNorm
                if (tid == 0) {
                    trace_mark(p, cta, l, TR_START);
                    if (p.trace) {
                        unsigned smid;
                        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
                        p.trace[(static_cast<size_t>(cta) * (p.n_layers + 1) + l) * TRACE_EVENTS + 9] = smid;
                    }
                }
                // both norms in one pass: y1 in xbuf[0, H), y2 in xbuf[H, 2H)
                if (p.arch_flags & AF_RMS_ADD) {
                    rms_norm_add_to_smem(x, p.residual_in, L->ln_w, H, p.norm_eps, sm.xbuf,
                                         cta == 0 ? p.residual_out : nullptr, sm.red, tid);
                } else {
                    layer_norm2_to_smem(x, xll, xep, ab, L->ln_w, L->ln_b, L->pln_w, L->pln_b, H, sm.xbuf,
                                        (ub > ua) ? sm.xbuf + H : nullptr, sm.red, tid);
                }
                if (tid == 0) trace_mark(p, cta, l, TR_LN_DONE);
                {
                    const __half* bq = L->b_qkv;
                    const __half* bu = L->b_up;
                    uint2* dq = p.qkv_ll;
                    const unsigned qep = ll_base + static_cast<unsigned>(l) + 1u;
                    float* dm = p.mid_f32;
                    __half* dm16 = p.mid_f16_out;
                    const int rowq0 = qa * GRAN, rowu0 = ua * GRAN;
                    co.rows_phase2(
                        qb - qa, ub - ua, KC1, sm.xbuf, (p.arch_flags & AF_RMS_ADD) ? sm.xbuf : sm.xbuf + H,
                        [&](int g, int r, float v) {
                            const int row = rowq0 + g * GRAN + r;
                            const float out = bq ? v + __half2float(__ldg(bq + row)) : v;
                            if (p.arch_flags & AF_QKV_PLANAR) {
                                // row of [Q_all; K_all; V_all] -> slot of the per-head [q; k; v] scratch
                                const int part = row / KVW, rem = row - part * KVW;
                                const int h = rem / D;
                                st_ll(dq + h * 3 * D + part * D + (rem - h * D), __float_as_uint(out), qep);
                            } else {
                                st_ll(dq + row, __float_as_uint(out), qep);
                            }
                        },
                        [&](int g, int r, float v) {
                            const int row = rowu0 + g * GRAN + r;
                            if (p.arch_flags & AF_SWIGLU) {  // raw gate / up values; combined where P3 stages them
                                dm[row] = v;
                                return;
                            }
                            const float pre = v + __half2float(__ldg(bu + row));
                            const float a = (p.arch_flags & AF_GELU_ERF) ? gelu_erf_f(pre) : gelu_tanh_f(pre);
                            dm[row] = a;
                            if (dm16) dm16[row] = __float2half_rn(a);
                        },
                        [&]() {});
                }
                // count this CTA past P1: its share of the MLP intermediate is written
                consumer_sync(NCTHR);
                if (tid == 0) {
                    __threadfence();
                    atomicAdd(p.sync + 3, 1u);
                    trace_mark(p, cta, l, TR_P1_DONE);
                }
                need_barrier = true;
            }

            // ------------------------------------------------------------ P2
            if (p.phase_mask & PH_P2) {
                // no grid barrier here: q/k/v words carry their epoch and are polled where they are used
                const unsigned pep = ll_base + static_cast<unsigned>(l) + 1u;  // epoch of this layer's records
                const QkvView qkv{p.qkv_ll, pep, p.qkv_any_epoch != 0, &ab};
                if (tid == 0) trace_mark(p, cta, l, TR_BAR1);
                // Empty cache (seq == 0): there are no items, so the head's owner CTA turns the
                // new token into the head's only partial.  Otherwise the CTA that streams the
                // head's last chunk folds the new token in (below).
                if (nch == 0 && warp == 0) {
                    for (int h = 0; h < NH; ++h) {
                        if (head_owner(h, NH, G) != cta) continue;
                        const int qi = h * 3 * D;
                        float s = 0.f;
                        for (int d = lane; d < D; d += 32) {
                            const float qd = rope_elem(qkv, qi, d, R, cosr, sinr) * qscale;
                            const __half k16 = __float2half_rn(rope_elem(qkv, qi + D, d, R, cosr, sinr));
                            const __half v16 = __float2half_rn(qkv.get(qi + 2 * D + d));
                            s = fmaf(qd, __half2float(k16), s);
                            const size_t off = static_cast<size_t>(seq) * KVW + h * D + d;
                            if (!(p.arch_flags & AF_NO_APPEND)) {
                                L->k_cache[off] = k16;
                                L->v_cache[off] = v16;
                            }
                            if (p.k_new) p.k_new[h * D + d] = k16;
                            if (p.v_new) p.v_new[h * D + d] = v16;
                            p.attn_new[h * PREC + d] = __half2float(v16);
                        }
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                        if (lane == 0) {
                            p.attn_new[h * PREC + D] = s;
                            p.attn_new[h * PREC + D + 1] = 1.0f;
                        }
                        __syncwarp();
                        if (lane == 0) publish_record(p.attn_new + h * PREC + D + 2, pep);
                    }
                }
                // cached rows: items [t2a, t2b), head-major
                const int hw = lane >> 4, l16 = lane & 15;
                const bool dim_ok = l16 * 8 < D;
                float* hbuf = sm.xbuf + p.aux_off + MAXHPC * 3 * D;  // hand-over buffer: [NCWARP][D]
                float* hml = hbuf + NCWARP * D;                      // [NCWARP][2]
                int cur_h = -1;
                float qreg[8], acc[8], m_run = -INFINITY, l_run = 0.f;
                const float* qpre = sm.xbuf + p.aux_off;
                const float* hq = qpre;

                // A head is finished (or this CTA's items end): the two half-warps of a warp join their
                // running states in registers, the warp leaves one slot in the hand-over buffer and
                // signals the helper warps, which combine the slots, fold in the new token, write and
                // stamp the record.  The consumers do not wait for that; only the next use of the
                // buffer waits (bounded) until the helpers have read the previous one.
                auto flush = [&]() {
                    const float mo = __shfl_xor_sync(0xffffffffu, m_run, 16);
                    const float lo = __shfl_xor_sync(0xffffffffu, l_run, 16);
                    const float M = fmaxf(m_run, mo);
                    const float ws = (m_run > -INFINITY) ? exp2f(m_run - M) : 0.f;
                    const float wo = (mo > -INFINITY) ? exp2f(mo - M) : 0.f;
                    float a2[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float ao = __shfl_xor_sync(0xffffffffu, acc[k], 16);
                        // the same expression on both half-warps: lower half first
                        a2[k] = (hw == 0) ? fmaf(acc[k], ws, ao * wo) : fmaf(ao, wo, acc[k] * ws);
                    }
                    const float l2 = (hw == 0) ? fmaf(l_run, ws, lo * wo) : fmaf(lo, wo, l_run * ws);
                    if (nflush > 0) mbar_wait(smem_u32(sm.pf_free), (nflush - 1u) & 1u, ab, ST_TIMEOUT_GRID);
                    if (hw == 0) {
                        if (dim_ok) {
                            *reinterpret_cast<float4*>(hbuf + warp * D + l16 * 8) = make_float4(a2[0], a2[1], a2[2], a2[3]);
                            *reinterpret_cast<float4*>(hbuf + warp * D + l16 * 8 + 4) = make_float4(a2[4], a2[5], a2[6], a2[7]);
                        }
                        if (l16 == 0) {
                            hml[warp * 2] = M;
                            hml[warp * 2 + 1] = l2;
                        }
                    }
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(sm.pf_ready));
                    ++nflush;
                };

                for (int t = t2a; t < t2b; ++t) {
                    const int h = t / nch, ch = t - h * nch;
                    if (h != cur_h) {
                        if (cur_h >= 0) flush();
                        cur_h = h;
                        // the helper warps staged q (and the new k, v where this CTA streams the
                        // head's last chunk) while P1 was still running
                        const int hi = h - t2a / nch;  // 0 or 1
                        hq = qpre + hi * 3 * D;
                        mbar_wait(smem_u32(sm.q_ready + hi), hi ? qpar1 : qpar0, ab, ST_TIMEOUT_GRID);
                        if (hi) qpar1 ^= 1u;
                        else qpar0 ^= 1u;
#pragma unroll
                        for (int k = 0; k < 8; ++k) {
                            qreg[k] = dim_ok ? hq[l16 * 8 + k] : 0.f;
                            acc[k] = 0.f;
                        }
                        m_run = -INFINITY;
                        l_run = 0.f;
                    }
                    const __half* kt = reinterpret_cast<const __half*>(co.wait_stage());
                    const int r0 = warp * (2 * KV_RPH) + hw * KV_RPH;
                    float s[KV_RPH];
#pragma unroll
                    for (int j = 0; j < KV_RPH; ++j) {
                        float d = 0.f;
                        if (dim_ok) {
                            const uint4 raw = *reinterpret_cast<const uint4*>(kt + (r0 + j) * D + l16 * 8);
                            const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const float2 f = __half22float2(h2[k]);
                                d = fmaf(f.x, qreg[2 * k], d);
                                d = fmaf(f.y, qreg[2 * k + 1], d);
                            }
                        }
                        s[j] = d;
                    }
                    co.release_stage();  // K tile consumed: scores are in registers
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
                        for (int j = 0; j < KV_RPH; ++j) s[j] += __shfl_xor_sync(0xffffffffu, s[j], o);
                    }
                    const int grow = ch * KV_TILE + r0;
                    float mx = m_run;
#pragma unroll
                    for (int j = 0; j < KV_RPH; ++j) {
                        if (grow + j >= seq) s[j] = -INFINITY;
                        mx = fmaxf(mx, s[j]);
                    }
                    float sc = 1.f;
                    if (mx > -INFINITY) {
                        sc = exp2f(m_run - mx);
                        m_run = mx;
#pragma unroll
                        for (int j = 0; j < KV_RPH; ++j) s[j] = (grow + j < seq) ? exp2f(s[j] - mx) : 0.f;
                    }
                    const __half* vt = reinterpret_cast<const __half*>(co.wait_stage());
                    if (mx > -INFINITY) {
                        l_run *= sc;
#pragma unroll
                        for (int k = 0; k < 8; ++k) acc[k] *= sc;
#pragma unroll
                        for (int j = 0; j < KV_RPH; ++j) {
                            if (grow + j < seq) {  // rows past the sequence may hold anything: never touch them
                                const float pj = s[j];
                                l_run += pj;
                                if (dim_ok) {
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
                    }
                    co.release_stage();
                    // (the token being decoded is folded in by the helper warps when they finish the partial)
                }
                if (cur_h >= 0) flush();
                if (tid == 0) trace_mark(p, cta, l, TR_P2_DONE);
                need_barrier = true;
            }

            // ------------------------------------------------------------ P3
            if (p.phase_mask & PH_P3) {
                // No grid barrier: the helper warps poll the attention partials record by record, and
                // one of their threads has watched the count of CTAs past P1 for the MLP intermediate.
                if (mid_wait) {
                    mbar_wait(smem_u32(sm.mid_ready), mparity, ab, ST_TIMEOUT_GRID);
                    mparity ^= 1u;
                }
                if (tid == 0) trace_mark(p, cta, l, TR_BAR2);
                // ---- this CTA's K slice of [mid ; attn] as fp32 in xbuf, chunk-major, MLP chunks
                // first.  The helper warps merge the attention partials into the chunks behind
                // them while the GEMV already runs over the MLP chunks.
                const int nmid = my3 - nattn;
                if (tid == 0) mbar_arrive(smem_u32(sm.h_go));
                if (mid_wait && (p.phase_mask & PH_P2)) {
                    // staged by helper warp 0 while this CTA was still in P2
                } else if (!(p.p3_flags & F3_MID_F16)) {
                    stage_mid(tid, NCTHR);
                } else {
                    for (int i0 = 0; i0 < nmid; i0 += 8) {
                        float v[8];
#pragma unroll
                        for (int ii = 0; ii < 8; ++ii) {
                            const int e = (me + (nattn + i0 + ii) * CS - KCo) * KCHUNK + tid;
                            v[ii] = (i0 + ii < nmid && e < F) ? __half2float(ld_cg_f16(p.mid_f16_in + e)) : 0.f;
                        }
#pragma unroll
                        for (int ii = 0; ii < 8; ++ii)
                            if (i0 + ii < nmid) sm.xbuf[(i0 + ii) * KCHUNK + tid] = v[ii];
                    }
                }
                // (3) what the epilogue adds to this thread's output row, fetched before the GEMV.  (Fetching it a
                // phase earlier, right after the LayerNorm, measured 1.2 % SLOWER per token: the thread stalls
                // there on the loads, and this point is not on the critical path.)
                float epi_add = 0.f;
                {
                    const int nrows_e = (g3b - g3a) * GRAN;
                    if (me + tid * CS < nrows_e) {
                        const int row = g3a * GRAN + me + tid * CS;
                        if (p.p3_flags & F3_ADD_BO) epi_add += __half2float(__ldg(L->b_o + row));
                        if (p.p3_flags & F3_ADD_BDOWN) epi_add += __half2float(__ldg(L->b_down + row));
                        if (p.p3_flags & F3_ADD_X)
                            epi_add += x ? __half2float(ld_cg_f16(x + row))
                                         : __half2float(__ushort_as_half(static_cast<unsigned short>(ld_ll(xll + row).x)));
                        if (p.extra_add_f16) epi_add += __half2float(ld_cg_f16(p.extra_add_f16 + row));
                    }
                }
                asm volatile("cp.async.wait_all;" ::: "memory");
                consumer_sync(NCTHR);
                if (tid == 0) trace_mark(p, cta, l, TR_X3_BUILT);

                const int cnt = g3b - g3a;
                const int nrows = cnt * GRAN;
                const int stride = MAX_P3_ROWS / CS;
                // every finished partial row goes straight from the lane that holds it to the CTA of the
                // cluster that owns the row (dsm.cuh); no CTA-wide barrier on the way
                if (cnt > 0) {
                    if (my3 > 0) {
                        float* rv = sm.recv;
                        co.rows_phase(cnt, my3, sm.xbuf,
                                      [&](int g, int r, float v) { dsm::scatter_row<CS>(rv, stride, me, g * GRAN + r, v); },
                                      nattn > 0 ? nmid : -1, smem_u32(sm.attn_ready), hparity);
                    } else {
                        for (int t = tid; t < nrows; t += NCTHR) dsm::scatter_row<CS>(sm.recv, stride, me, t, 0.f);
                    }
                }
                else if (nattn > 0) mbar_wait(smem_u32(sm.attn_ready), hparity, ab, ST_TIMEOUT_FULL);  // keep phases paired
                hparity ^= 1u;
                dsm::exchange_arrive<CS>(sm.xbar, me, lane);
                if (tid == 0) trace_mark(p, cta, l, TR_P3_GEMV);
                dsm::exchange_wait(sm.xbar, xparity, ab);
                xparity ^= 1u;
                // one output row per thread at most (MAX_P3_ROWS / CS <= consumer threads)
                if (p.tp_size <= 1) {
                    if (me + tid * CS < nrows) {
                        const int row = g3a * GRAN + me + tid * CS;
                        store_y(row, dsm::tree_sum<CS>(sm.recv, stride, tid) + epi_add);
                    }
                } else {
                    // Tensor parallel: what this CTA holds is one rank's partial of its rows.  The
                    // same thread of the same CTA owns the same row on every rank, so the all-reduce
                    // is a thread-to-thread exchange: store my partial row, tagged with this layer's
                    // epoch, into every peer's buffer (8-byte stores over NVLink), wait (bounded)
                    // for the N-1 counterparts' words to show the epoch, add the N partials in
                    // rank order in fp32.  Slots alternate with the exchange's epoch parity -- consecutive
                    // exchanges, also across launches and for any layer count, differ in it -- so a slot is
                    // rewritten only after its reader has sent its next word.
                    const TpLayout tl{H, p.tp_size};
                    const unsigned tp_epoch = tp_base + static_cast<unsigned>(l) + 1u;
                    const int parity = static_cast<int>(tp_epoch & 1u);
                    if (me + tid * CS < nrows) {
                        const int row = g3a * GRAN + me + tid * CS;
                        // the word's place in a slot: by row, or (packed) the cluster's row range re-ordered so that
                        // the words of one CTA are contiguous and its threads' peer stores leave as whole lines
                        // -- the same permutation on every rank, since the partition is the same
                        int word = row;
                        if (p.tp_packed) {
                            word = g3a * GRAN + tid;
                            for (int m = 0; m < me; ++m) word += (nrows - m + CS - 1) / CS;
                        }
                        const float mine = dsm::tree_sum<CS>(sm.recv, stride, tid);
                        for (int r = 0; r < p.tp_size; ++r)
                            if (r != p.tp_rank)
                                st_ll_sys(p.tp_peer[r] + tl.partial_off(parity, p.tp_rank) + static_cast<size_t>(word) * 8,
                                      __float_as_uint(mine), tp_epoch);
                        // (no fence after them: a system-scope fence here measured 1.5 us SLOWER per exchange)
                        // all counterparts' words in flight at once; re-read (bounded) until every epoch matches
                        const unsigned char* mybuf = p.tp_peer[p.tp_rank] + static_cast<size_t>(word) * 8;
                        uint2 w[MAX_TP];
                        auto fetch = [&]() {
                            bool ok = true;
#pragma unroll
                            for (int r = 0; r < MAX_TP; ++r) {
                                if (r < p.tp_size && r != p.tp_rank) {
                                    w[r] = ld_ll_sys(mybuf + tl.partial_off(parity, r));
                                    ok = ok && (w[r].y == tp_epoch);
                                }
                            }
                            return ok;
                        };
                        if (!fetch()) wait_bounded<POLL_BACKOFF_NS>(fetch, ab, ST_TIMEOUT_PEER);
                        float sum = 0.f;
#pragma unroll
                        for (int r = 0; r < MAX_TP; ++r)
                            if (r < p.tp_size) sum += (r == p.tp_rank) ? mine : __uint_as_float(w[r].x);
                        store_y(row, sum + epi_add);
                    }
                }
                if (tid == 0) trace_mark(p, cta, l, TR_P3_DONE);
                need_barrier = true;
            }
        }

        // ---------------------------------------------------------------- P4
        if (p.phase_mask & PH_P4) {
            const TailDesc* Tl = p.tail;
            const __half* x = (p.n_layers > 0) ? p.out : x_first;
            if (need_barrier) grid_barrier(p.sync, epoch, G, tid, ab);
            if (tid == 0) trace_mark(p, cta, p.n_layers, TR_START);
            float best = -INFINITY;
            int best_i = 0x7fffffff;
            if (g4b > g4a) {
                layer_norm_to_smem(x, Tl->fln_w, Tl->fln_b, H, sm.xbuf, sm.red, tid, false);
                if (tid == 0) trace_mark(p, cta, p.n_layers, TR_LN_DONE);
                const int row0 = g4a * GRAN, V = Tl->vocab;
                float* lg = p.logits;
                co.rows_phase2(
                    0, g4b - g4a, KC1, sm.xbuf, sm.xbuf, [](int, int, float) {},
                    [&](int g, int r, float v) {
                        const int row = row0 + g * GRAN + r;
                        if (row < V) {
                            if (lg) lg[row] = v;
                            if (v > best || (v == best && row < best_i)) {
                                best = v;
                                best_i = row;
                            }
                        }
                    },
                    [] {});
            }
            if (tid == 0) trace_mark(p, cta, p.n_layers, TR_P1_DONE);
            // arg-max: warp, then CTA, then (after a grid barrier) CTA 0
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, best, o);
                const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
                if (ov > best || (ov == best && oi < best_i)) {
                    best = ov;
                    best_i = oi;
                }
            }
            consumer_sync(NCTHR);
            int* redi = reinterpret_cast<int*>(sm.red + 16);
            if (lane == 0) {
                sm.red[warp] = best;
                redi[warp] = best_i;
            }
            consumer_sync(NCTHR);
            if (tid == 0) {
                for (int i = 1; i < NCWARP; ++i) {
                    if (sm.red[i] > best || (sm.red[i] == best && redi[i] < best_i)) {
                        best = sm.red[i];
                        best_i = redi[i];
                    }
                }
                p.amax_val[cta] = best;
                p.amax_idx[cta] = best_i;
            }
            grid_barrier(p.sync, epoch, G, tid, ab);
            if (tid == 0) trace_mark(p, cta, p.n_layers, TR_BAR1);
            if (cta == 0 && warp == 0) {
                float b = -INFINITY;
                int bi = 0x7fffffff;
                for (int i = lane; i < G; i += 32) {
                    const float v = __ldcg(p.amax_val + i);
                    const int vi = __ldcg(p.amax_idx + i);
                    if (v > b || (v == b && vi < bi)) {
                        b = v;
                        bi = vi;
                    }
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, b, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (ov > b || (ov == b && oi < bi)) {
                        b = ov;
                        bi = oi;
                    }
                }
                bi += p.vocab_offset;
                if (p.tp_size > 1) {
                    // vocabulary shards: every rank sends its (max, index) to all ranks and all
                    // pick the same winner (largest logit, lowest index on ties)
                    const TpLayout tl{H, p.tp_size};
                    const unsigned tp_epoch = tp_base + static_cast<unsigned>(p.n_layers) + 1u;
                    const int parity = static_cast<int>(__ldcg(p.tp_epoch_base + 1) & 1u);  // launches of this decoder so far
                    if (lane < p.tp_size && lane != p.tp_rank) {
                        unsigned char* dst = p.tp_peer[lane] + tl.pairs_off(parity, p.tp_rank);
                        st_ll_sys(dst, __float_as_uint(b), tp_epoch);
                        st_ll_sys(dst + 8, static_cast<unsigned>(bi), tp_epoch);
                    }
                    float rb = -INFINITY;
                    int rbi = 0x7fffffff;
                    if (lane == p.tp_rank) {
                        rb = b;
                        rbi = bi;
                    } else if (lane < p.tp_size) {
                        const unsigned char* src = p.tp_peer[p.tp_rank] + tl.pairs_off(parity, lane);
                        rb = __uint_as_float(wait_ll_sys(src, tp_epoch, ab));
                        rbi = static_cast<int>(wait_ll_sys(src + 8, tp_epoch, ab));
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) {
                        const float ov = __shfl_xor_sync(0xffffffffu, rb, o);
                        const int oi = __shfl_xor_sync(0xffffffffu, rbi, o);
                        if (ov > rb || (ov == rb && oi < rbi)) {
                            rb = ov;
                            rbi = oi;
                        }
                    }
                    b = rb;
                    bi = rbi;
                }
                if (lane == 0) {
                    if (p.token_out) *p.token_out = bi;
                    p.amax_val[0] = b;  // winner's logit
                    p.amax_idx[0] = bi;
                }
            }
        }

        // ---- leave: count out; the last CTA re-arms the barrier words
        {
            consumer_sync(NCTHR);
            if (tid == 0) {
                __threadfence();
                const unsigned old = atomicAdd(p.sync + 1, 1u);
                if (old == static_cast<unsigned>(G) - 1u) {
                    p.sync[0] = 0u;
                    p.sync[1] = 0u;
                    p.sync[3] = 0u;
                    *p.epoch_base = *p.epoch_base + static_cast<unsigned>(p.n_layers) + 2u;
                    if (p.seq_inc) *p.seq_inc = seq + 1;
                    if (p.tp_size > 1) {
                        p.tp_epoch_base[0] = p.tp_epoch_base[0] + static_cast<unsigned>(p.n_layers) + 2u;
                        p.tp_epoch_base[1] = p.tp_epoch_base[1] + 1u;
                    }
                    __threadfence();
                }
            }
        }
    }
    // no CTA leaves while a peer may still store into its shared memory
    __syncthreads();
    if constexpr (CS > 1) dsm::cluster_sync_all();
}

template <int D, int CS>
__global__ void __launch_bounds__(NTHREADS, 1) fused_decode_kernel(const __grid_constant__ Params p) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    decode_body<D, CS>(p, p.kv_maps, smem_raw);
}

// Several parameter blocks as ONE launch (a stack of layers whose blocks differ in kind: the Llama attention
// and SwiGLU MLP blocks), in order.  Each block runs exactly as its own launch would -- barriers initialised,
// work split derived, epochs read -- from a copy of its parameters in shared memory; between two blocks all CTAs
// meet at a sense-reversing grid barrier (bar[0] arrivals, bar[1] generation), which orders the next block
// behind everything the previous one wrote, its bookkeeping words included.  What a launch boundary costs beyond
// that (drain, launch, CTA start-up) is gone.
struct MultiArgs {
    const Params* blocks;   // [n_blocks] in global memory
    int n_blocks;
    int params_off;         // byte offset of the parameter copy inside dynamic shared memory (beyond every block's own use)
    unsigned* bar;          // two words, zero before the first launch
    int* status;
};
template <int D, int CS>
__global__ void __launch_bounds__(NTHREADS, 1) fused_decode_multi_kernel(const __grid_constant__ MultiArgs a) {
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    static_assert(sizeof(Params) % 16 == 0, "the parameter block is copied in 16-byte pieces");
    Params* sp = reinterpret_cast<Params*>(smem_raw + a.params_off);
    const int tid = threadIdx.x;
    for (int b = 0; b < a.n_blocks; ++b) {
        {
            const uint4* src = reinterpret_cast<const uint4*>(a.blocks + b);
            uint4* dst = reinterpret_cast<uint4*>(sp);
            for (int i = tid; i < static_cast<int>(sizeof(Params) / 16); i += NTHREADS) dst[i] = __ldg(src + i);
        }
        __syncthreads();
        decode_body<D, CS>(*sp, a.blocks[b].kv_maps, smem_raw);
        // every thread is out of the block; peers' remote arrivals have landed before the barriers are re-made
        __syncthreads();
        if constexpr (CS > 1) dsm::cluster_sync_all();
        if (tid == 0) {
            // the next block initialises its barriers afresh: invalidate this block's first
            const Smem sm = carve(smem_raw, sp->nstage, sp->xbuf_floats);
            for (int s = 0; s < sp->nstage; ++s) {
                mbar_inval(smem_u32(sm.full + s));
                mbar_inval(smem_u32(sm.empty + s));
            }
            for (int i = 0; i < 9; ++i) mbar_inval(smem_u32(sm.xbar + i));
        }
        __syncthreads();
        if (b + 1 < a.n_blocks) {
            if (tid == 0) {
                const unsigned gen = ld_acquire_u32(a.bar + 1);
                __threadfence();
                const unsigned old = atomicAdd(a.bar, 1u);
                if (old == gridDim.x - 1u) {
                    a.bar[0] = 0u;
                    __threadfence();
                    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(a.bar + 1), "r"(gen + 1u) : "memory");
                } else {
                    // bounded like every wait of this kernel: on a timeout the status word says so and the
                    // remaining blocks run on (their own waits will give up as well)
                    const unsigned long long t0 = globaltimer_ns();
                    while (ld_acquire_u32(a.bar + 1) == gen) {
                        __nanosleep(64);
                        if (globaltimer_ns() - t0 > wait_limit_ns(ST_TIMEOUT_GRID)) {
                            atomicCAS(a.status, 0, ST_TIMEOUT_GRID);
                            break;
                        }
                    }
                }
                __threadfence();
            }
            __syncthreads();
        }
    }
}

}  // namespace cfb
