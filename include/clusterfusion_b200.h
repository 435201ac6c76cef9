/* clusterfusion_b200.h — C ABI of the B200 (sm_100a) fused Pythia/GPT-NeoX decode path.
 *
 * Every entry point is `extern "C"`, takes plain device pointers and sizes, and
 * returns 0 on success or a negative CF_ERR_* code; cf_last_error() then gives a
 * thread-local message.  All tensors are contiguous fp16 on the current CUDA
 * device unless stated otherwise; cos/sin are fp32.  `stream` is a cudaStream_t
 * passed as void* (NULL = legacy default stream).  Nothing here synchronises the
 * device unless its comment says so.
 *
 * Each declaration cites the interface of the reference project
 * (superk668/ClusterFusionPlus) that it replaces, as file:line.
 */
#ifndef CLUSTERFUSION_B200_H_
#define CLUSTERFUSION_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CF_OK 0
#define CF_ERR_INVALID (-1)   /* bad argument (shape, alignment, range, unknown id) */
#define CF_ERR_CUDA (-2)      /* a CUDA runtime / driver call failed */
#define CF_ERR_DEVICE (-3)    /* the kernel reported a device-side status (timeout, bad seq_len) */
#define CF_ERR_UNSUPPORTED (-4)

/* Model ids of the reference's per-model entry points. */
#define CF_PYTHIA_2B8 0   /* include/5090/pythia_2b8/config.h:6-12  */
#define CF_PYTHIA_6B9 1   /* include/5090/pythia_6b9/config.h:6-12  */

/* Geometry of (a shard of) a GPT-NeoX style model.  `heads` and `ffn` are what
 * THIS rank holds; hidden is always the full width. */
typedef struct CfDims {
    int hidden;    /* HIDDEN_DIM */
    int heads;     /* HEAD_NUM (local) */
    int head_dim;  /* HEAD_DIM: 80 or 128 */
    int rotary;    /* ROTARY_DIM */
    int ffn;       /* FFN_DIM (local) */
    int vocab;     /* LM-head rows held by this rank (0 = no tail) */
} CfDims;

/* The 12 parameter tensors of one layer; argument order of
 * include/pybind.cpp:109-129 (pythia_*_decoder_layer_sm120). */
typedef struct CfLayerWeights {
    const void* qkv_weight;      /* [3*heads*head_dim, hidden], rows interleaved per head [Q_h;K_h;V_h] */
    const void* qkv_bias;        /* [3*heads*head_dim] */
    const void* o_weight;        /* [hidden, heads*head_dim] */
    const void* o_bias;          /* [hidden] */
    const void* ln_weight;       /* [hidden] */
    const void* ln_bias;
    const void* post_ln_weight;  /* [hidden] */
    const void* post_ln_bias;
    const void* mlp_up_weight;   /* [ffn, hidden] */
    const void* mlp_up_bias;     /* [ffn] */
    const void* mlp_down_weight; /* [hidden, ffn] */
    const void* mlp_down_bias;   /* [hidden] */
} CfLayerWeights;

/* Per-call tensors of one layer call. */
typedef struct CfLayerIO {
    const void* input;       /* [1, hidden] */
    void* k_cache;           /* [kv_rows, heads*head_dim]; row seq_len is written */
    void* v_cache;
    int64_t kv_rows;         /* rows allocated in each cache; seq_len must be < kv_rows */
    const float* cos;        /* fp32, first `rotary` entries used */
    const float* sin;
    void* output;            /* [1, hidden] */
    void* k_new;             /* [1, heads, head_dim] or NULL */
    void* v_new;
    void* attn_output;       /* attention_only: [1, hidden] */
    void* mlp_intermediate;  /* attention_only: [ffn] */
} CfLayerIO;

const char* cf_last_error(void);

/* Geometry of a built-in model id. */
int cf_model_dims(int model, CfDims* out);

/* Launch geometry the library chose on the current device: SM count, CTAs in the
 * persistent grid, cluster size, TMA ring stages for `model`. */
int cf_launch_info(int model, int* sm_count, int* grid, int* cluster, int* stages, int* smem_bytes);

/* Reads the device status words of the current device -- the shared workspace of the layer
 * calls, every decoder, and the static scratch of cf_pythia_decoder_layer_noalloc
 * (synchronises the device) -- clears what was set and re-arms the barrier words.
 * *status = 0 when every launch so far finished normally; otherwise the call returns
 * CF_ERR_DEVICE and *status is 1-2 TMA ring, 3 grid barrier / flag wait, 4 cluster exchange,
 * 5 bad seq_len, 6 drain, 7 tensor-parallel peer never answered. */
int cf_get_status(int* status);

/* Fused decoder layer, one token at batch 1.  The first call with a given set of tensors
 * builds and uploads their descriptor (tensor maps), so it allocates and cannot be recorded
 * into a stream capture (CF_ERR_INVALID while capturing); later calls with the same tensors
 * can.  The same holds for the split, attention_only, mlp_only and Llama entry points.
 * Replaces pythia_2b8_decoder_layer_sm120 / pythia_6b9_decoder_layer_sm120
 * (include/pybind.cpp:109-129,198-218; include/5090/pythia_6b9/pythia_kernel_dispatch.cu:4-236). */
int cf_pythia_decoder_layer(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, void* stream);

/* Same result (bit for bit) from two launches with the kernel boundary in place
 * of the second grid barrier.
 * Replaces pythia_2b8_decoder_layer_split_sm120 (include/pybind.cpp:132-151;
 * include/5090/pythia_2b8/pythia_kernel_dispatch_split.cu:18-218). */
int cf_pythia_decoder_layer_split(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len,
                                  void* stream);

/* The fused decoder layer for callers that cannot allocate device memory at the point
 * of the call: code running under a memory pool that owns the whole GPU (inference
 * servers that pre-reserve all of HBM, so a late cudaMalloc fails or fragments), and
 * callers inside a region where allocation is forbidden (e.g. they already hold the
 * allocator's lock).  Same arguments, same result bits as cf_pythia_decoder_layer, but
 * this entry point performs no cudaMalloc / cudaFree and calls no allocating routine:
 * its scratch (fp32 QKV and MLP intermediates, attention partials, barrier words and
 * the layer descriptor with its tensor maps) lives in a static __device__ array of
 * 522,112 bytes that every GPU loading the library holds until exit.
 *   Limits: the built-in models only (at most 32 heads, 4096 QKV columns, ffn 16384)
 *   on at most 160 CTAs; anything larger is rejected with CF_ERR_UNSUPPORTED.
 *   The first call on a device looks up the array's device address and the launch
 *   geometry; make that first call outside any stream capture.  So must be every call
 *   whose tensors differ from the previous call's: it uploads a new descriptor, which a
 *   capture cannot record (such a call fails with CF_ERR_INVALID while capturing).
 *   All calls on a device share the one array and it keeps the previous call's
 *   contents (the words that must start at zero are cleared on `stream` each call):
 *   two calls whose kernels overlap on the GPU (different streams) race.
 *   A device-side failure of these launches (a wait that ran out, a bad seq_len) is
 *   kept in the array's status word until cf_get_status reports and clears it.
 * No counterpart in the reference (its dispatcher allocates five tensors per call:
 * include/5090/pythia_6b9/pythia_kernel_dispatch.cu:31-39). */
int cf_pythia_decoder_layer_noalloc(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len,
                                    void* stream);

/* Llama-2-7B attention block, one token at batch 1 (hidden 4096, 32 heads x 128, full NeoX
 * RoPE, no biases): residual_out = input + residual (fp16; residual may be NULL = zeros);
 * h = RMSNorm(residual_out, rms_input_weight, eps); q,k,v = weight_qkv h with rows laid out
 * [Q of all heads; K of all heads; V of all heads]; rotate-half RoPE with cos/sin[128];
 * attention over the seq_len rows of k_cache / v_cache ([seq_len, 4096], NOT written) plus the
 * new token; output = weight_o attn (weight_o [4096, 4096] in nn.Linear layout).  k_new is
 * post-RoPE, [32,128].  residual_out must not alias residual.
 * Replaces llama_decoder_layer_sglang_sm120 (include/pybind.cpp:75-86;
 * include/5090/llama/llama_kernel_sglang_dispatch.cu:4-151; kernel_sglang.cuh:20-634).
 * The paged batch entry point is cf_llama_decoder_layer_batch_sglang below; the reference's
 * transposed-weight llama_decoder_layer (include/pybind.cpp:66-74) is not provided: it computes the same
 * block from weights stored [in, out], a layout none of the reference's tests or benchmarks exercise; a
 * caller that holds such weights transposes them once when loading. */
int cf_llama_decoder_layer_sglang(const void* input, const void* residual, const void* weight_qkv,
                                  const void* weight_o, const void* k_cache, const void* v_cache, int64_t seq_len,
                                  const void* rms_input_weight, float eps, const float* cos, const float* sin,
                                  void* output, void* residual_out, void* k_new, void* v_new, void* stream);

/* The SwiGLU MLP block that follows the attention block in a Llama-2-7B layer, with the same
 * fused-add front:  residual_out = input + residual (fp16);  y = RMSNorm(residual_out, eps) * rms_weight;
 * output = (silu(y Wg^T) * (y Wu^T)) Wd^T.   gate_up_weight is [2*ffn, 4096] with the gate rows first
 * (the merged gate_up_proj of serving stacks), down_weight [4096, ffn]; no biases.  `residual` may be
 * NULL.  The reference's Llama kernels stop after the attention block and leave this block to the
 * caller (tests/test_llama.py:108-110 has it commented out); a full Llama layer needs it. */
int cf_llama_mlp_sglang(const void* input, const void* residual, const void* gate_up_weight, const void* down_weight,
                        const void* rms_weight, float eps, int64_t ffn, void* output, void* residual_out, void* stream);

/* Several layer-level calls as ONE launch.  Between cf_batch_begin() and cf_batch_end(stream) the layer-level
 * entry points called on this thread (cf_pythia_*, cf_*_graph_decode_step, cf_llama_decoder_layer_sglang,
 * cf_llama_mlp_sglang; head_dim 128 models) validate and prepare their launch as usual but do not launch; their
 * stream arguments are ignored.  cf_batch_end launches one persistent kernel on `stream` that runs the recorded
 * blocks in call order, each exactly as its own launch would have run, with a grid barrier in between: what a
 * launch boundary costs beyond that is gone (a 32-layer Llama stack is 64 blocks).  The blocks' parameters are
 * uploaded only when they differ from the previous batch's, so an unchanged batch can be captured into a CUDA
 * graph; one that changed is refused during capture (CF_ERR_UNSUPPORTED).  cf_batch_abort() drops an open batch.
 * Calls that cannot be part of a batch (the whole-token decoder, tensor-parallel launches, the batched Llama
 * blocks, which are another kernel) fail or launch at once as documented for them.  The reference has no
 * counterpart: its callers pay one launch per layer (tests/benchmark_decode_6b9.py:133-198). */
int cf_batch_begin(void);
int cf_batch_end(void* stream);
int cf_batch_abort(void);

/* Llama-2-7B attention block for a BATCH of 1..16 decode sequences over a paged KV pool, one launch.
 * Per sequence b: residual_output[b] = input[b] + residual[b] (fp16; residual may be NULL);
 * h = RMSNorm(residual_output[b], rms_input_weight, eps); q,k,v = weight_qkv h (rows [Q of all heads;
 * K of all heads; V of all heads]); rotate-half RoPE with the angles of row positions[b] of cos_sin
 * ([positions, 128] fp32: 64 cosines, then 64 sines).  Sequence b owns the pool rows
 * paged_kv_indices[paged_kv_indptr[b] .. paged_kv_indptr[b+1]) -- one row = one token, [4096] fp16 --
 * of the pools k_cache_ptrs[layer_id] / v_cache_ptrs[layer_id] (device arrays of device pointers): the LAST
 * entry is the slot the new key / value are written to, the entries before it are the history that is
 * attended to (plus the new token); every sequence needs at least that one entry.
 * output[b] = weight_o attention(b).  All tensors [batch, 4096] fp16 unless said otherwise; indptr /
 * indices int32, positions int64.  The weights are streamed once for the whole batch: the projections run
 * as skinny GEMMs on the tensor cores (tcgen05), the rest as in the batch-1 block.  The first call on a
 * device allocates 2.3 MB of scratch (not capturable); calls on one device share it and must not overlap.
 * Replaces llama_decoder_layer_batch_sglang_sm120 (include/pybind.cpp:90-106,282;
 * include/5090/llama/llama_kernel_batch_sglang_dispatch.cu:6-111; kernel_batch_sglang.cuh:43-664). */
int cf_llama_decoder_layer_batch_sglang(void* output, void* residual_output, const void* input, const void* residual,
                                        const void* weight_qkv, const void* weight_o, const int* paged_kv_indptr,
                                        const int* paged_kv_indices, const uint64_t* k_cache_ptrs,
                                        const uint64_t* v_cache_ptrs, int layer_id, const void* rms_input_weight, float eps,
                                        const int64_t* positions, const float* cos_sin, int64_t batch, void* stream);

/* The SwiGLU MLP block (see cf_llama_mlp_sglang) for a batch of 1..16 rows, weights streamed once:
 * residual_out[b] = input[b] + residual[b]; output[b] = (silu(y Wg^T) * (y Wu^T)) Wd^T with
 * y = RMSNorm(residual_out[b]) * rms_weight.  ffn must be a multiple of 64.  No counterpart in the
 * reference, which leaves the MLP to its caller (tests/test_llama.py:108-110). */
int cf_llama_mlp_batch_sglang(const void* input, const void* residual, const void* gate_up_weight, const void* down_weight,
                              const void* rms_weight, float eps, int64_t ffn, int64_t batch, void* output,
                              void* residual_out, void* stream);

/* Diagnostic: while a buffer is set (uint64 [256][16] or larger), every batched Llama launch on the current device
 * stamps the nanosecond timer of each CTA at its phase boundaries (start, after the norm, after each grid barrier and
 * each phase, end).  NULL switches it off.  No counterpart in the reference. */
int cf_debug_set_llama_batch_trace(void* device_buffer, int64_t n_slots);

/* Diagnostic: run any subset of the layer's phases (bit 0: LayerNorm + QKV + MLP-up,
 * bit 1: RoPE + KV append + attention, bit 2: O-proj + MLP-down + residual) in one
 * launch, reading what earlier phases left in the library's scratch.  Used by the
 * profiling scripts to time phases in isolation; no counterpart in the reference. */
int cf_debug_run_phases(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, int phase_mask,
                        void* stream);

/* Diagnostic: while a buffer is set, every launch on the current device stamps the
 * nanosecond timer at its phase boundaries into it, laid out
 * [CTA][layer (n_layers + 1 rows)][16 events] uint64; n_slots = its length in
 * elements; a launch that would not fit leaves it untouched.  NULL switches it
 * off.  No counterpart in the reference. */
int cf_debug_set_trace(void* device_buffer, int64_t n_slots);

/* Diagnostic: the streaming ceiling of the decode kernel's own machinery.  One launch of the
 * persistent grid streams matrix [rows, cols] fp16 (rows a multiple of 8, cols a multiple of 256, at
 * most 4096) through the same TMA ring, producer and row-GEMV consumers as the LM-head phase, with
 * nothing to wait for but the data: rows are dotted with x [cols] and discarded (touch_only != 0:
 * the consumers take and release each stage without the arithmetic).  rows * cols * 2 bytes over the
 * launch time is the read bandwidth the kernel's structure can reach.  scratch_desc: 1 KB of device
 * memory, 128-byte aligned, owned by the caller (the descriptor is uploaded there; the call
 * synchronises `stream` once).  No counterpart in the reference. */
int cf_debug_stream_rows(const void* matrix, int64_t rows, int64_t cols, const void* x, int touch_only,
                         void* scratch_desc, void* stream);

/* Diagnostic: device address and size of the static scratch of cf_pythia_decoder_layer_noalloc
 * on the current device, and the byte offset of its status word (tests write a code there from
 * the host to check that cf_get_status reports it).  Allocates nothing. */
int cf_debug_noalloc_scratch(void** base, int64_t* bytes, int64_t* status_offset);

/* Attention half: io->attn_output = dense(attention) + o_bias, io->mlp_intermediate =
 * gelu(up(post_ln(x))), io->k_new / io->v_new.  mlp_down_* of `w` may be NULL.
 * Replaces pythia_2b8_attention_only_sm120 (include/pybind.cpp:154-171;
 * pythia_kernel_dispatch_split.cu:225-359). */
int cf_pythia_attention_only(int model, const CfLayerWeights* w, const CfLayerIO* io, int64_t seq_len, void* stream);

/* MLP half: output = input + attn_output + down(mlp_intermediate) + down_bias.
 * Replaces pythia_2b8_mlp_only_sm120 (include/pybind.cpp:174-180;
 * pythia_kernel_dispatch_split.cu:364-426). */
int cf_pythia_mlp_only(int model, const void* input, const void* attn_output, const void* mlp_intermediate,
                       const void* mlp_down_weight, const void* mlp_down_bias, void* output, void* stream);

/* Persistent per-layer context: tensor maps sized to max_seq_len and static
 * output buffers owned by the library.
 * Replaces pythia_*_create_graph_context_sm120 (include/pybind.cpp:206-215;
 * include/5090/pythia_6b9/pythia_kernel_dispatch_graph.cu:77-206). */
int cf_pythia_create_graph_context(int model, int64_t context_id, void* k_cache, void* v_cache,
                                   const void* weight_qkv, const void* weight_o, const void* mlp_up_weight,
                                   const void* mlp_down_weight, int64_t max_seq_len);

/* Small per-step tensors of graph_decode_step, order of include/pybind.cpp:217-233. */
typedef struct CfStepArgs {
    const void* input;
    const void* ln_weight;
    const void* ln_bias;
    const void* qkv_bias;
    const void* o_bias;
    const float* cos;
    const float* sin;
    void* k_cache;
    void* v_cache;
    const void* post_ln_weight;
    const void* post_ln_bias;
    const void* mlp_up_bias;
    const void* mlp_down_bias;
} CfStepArgs;

/* One layer step through a context.  *output, *k_new, *v_new receive pointers to
 * the context's static buffers ([hidden], [heads*head_dim] x2), valid until the
 * context is destroyed and overwritten by the next step.
 * Replaces pythia_*_graph_decode_step_sm120 (include/pybind.cpp:217-233;
 * pythia_kernel_dispatch_graph.cu:212-287). */
int cf_pythia_graph_decode_step(int model, int64_t context_id, const CfStepArgs* a, int64_t seq_len, void* stream,
                                void** output, void** k_new, void** v_new);

/* Optional: make a context replayable inside a captured CUDA graph.  With a
 * device-resident sequence length and a RoPE table ([rows, stride] fp32 each) the
 * step reads both from device memory, so the seq_len / cos / sin arguments of
 * cf_pythia_graph_decode_step are ignored.  NULL pointers switch back.
 * (The reference bakes seq_len into the launch: pythia_kernel_dispatch_graph.cu:260-261.) */
int cf_pythia_graph_set_device_state(int model, int64_t context_id, const int* seq_len_dev, const float* cos_table,
                                     const float* sin_table, int64_t table_stride);

/* Replaces pythia_*_destroy_graph_context_sm120 (pythia_kernel_dispatch_graph.cu:292-294). */
int cf_pythia_destroy_graph_context(int model, int64_t context_id);

/* ---------------------------------------------------------------------------
 * Whole-model greedy decoder: embedding gather -> n_layers fused layers ->
 * final LayerNorm -> LM head -> argmax, one persistent launch per token,
 * capture-safe (no allocation, no host sync, sequence length and token id live
 * in device memory).  The reference runs this loop in Python around its layer
 * op (tests/benchmark_decode_6b9.py:133-198).
 * ------------------------------------------------------------------------- */
typedef struct CfDecoderConfig {
    CfDims dims;
    int n_layers;
    int64_t max_seq_len;     /* rows of every KV cache */
    int tp_size;             /* 1 = single GPU */
    int tp_rank;
    const float* cos_table;  /* [max_seq_len, rotary] fp32 */
    const float* sin_table;
    int flags;               /* CF_DECODER_* */
} CfDecoderConfig;

/* MLP activation is the exact (erf) GELU, as in the published Pythia checkpoints
 * (hidden_act "gelu"), instead of the tanh form the reference kernels hard-code
 * (include/5090/pythia_6b9/kernel.cuh:39-54). */
#define CF_DECODER_GELU_ERF 1

typedef struct CfHeadWeights {
    const void* embed_in;         /* [vocab_total, hidden] */
    const void* final_ln_weight;  /* [hidden] */
    const void* final_ln_bias;
    const void* embed_out;        /* [vocab (local), hidden] */
    int vocab_offset;             /* first vocabulary row held by this rank */
} CfHeadWeights;

int cf_decoder_create(const CfDecoderConfig* cfg, int64_t* handle);
int cf_decoder_set_layer(int64_t handle, int layer, const CfLayerWeights* w, void* k_cache, void* v_cache);
int cf_decoder_set_head(int64_t handle, const CfHeadWeights* head);
/* Uploads descriptors; must be called once after the setters, outside capture. */
int cf_decoder_finalize(int64_t handle);
/* Device-resident state: token id (in/out), sequence length, logits [vocab] fp32,
 * last hidden state [hidden] fp16, and (tensor-parallel) the fp16 partial [hidden]
 * that the caller all-reduces and the (max logit, index) pair of this shard. */
int cf_decoder_state(int64_t handle, int** token, int** seq_len, float** logits, void** hidden, void** partial,
                     float** shard_max, int** shard_idx);
/* Enqueue one whole token on `stream` (tp_size == 1, or a connected tensor-parallel decoder). */
int cf_decoder_step(int64_t handle, void* stream);
/* Tensor-parallel decoders (tp_size 2..8, one process per GPU of one NVLink-connected box):
 * cf_decoder_step then runs the whole token as ONE launch per rank, with the per-layer
 * all-reduce done inside the kernel by peer stores into the other ranks' exchange buffers
 * (no NCCL on the data path).  Set-up, once: every rank calls cf_decoder_tp_export (allocates
 * its exchange buffer, returns a 64-byte CUDA IPC handle), the host program all-gathers the
 * handles in rank order (tp_size x 64 bytes) and passes them to cf_decoder_tp_connect.  All
 * ranks must then enqueue the same sequence of cf_decoder_step calls.  A peer that never shows
 * up ends the local wait after 1.0 s with device status 7. */
int cf_decoder_tp_export(int64_t handle, void* ipc_handle_out);
int cf_decoder_tp_connect(int64_t handle, const void* all_handles);
/* Same, for a host program that drives all GPUs from ONE process with peer access enabled
 * (cudaDeviceEnablePeerAccess): after cf_decoder_tp_export on every decoder, read each one's
 * exchange buffer with cf_decoder_tp_buffer and hand every decoder the table of tp_size device
 * pointers in rank order (the entry of its own rank is ignored). */
int cf_decoder_tp_buffer(int64_t handle, void** buffer, int64_t* bytes);
int cf_decoder_tp_connect_pointers(int64_t handle, void* const* peer_buffers);
/* Tensor-parallel pieces for callers that bring their own all-reduce (NCCL), enqueued per layer around the caller's all-reduce of
 * `partial`: layer_partial -> all-reduce(partial) -> layer_finish; then tail. */
int cf_decoder_layer_partial(int64_t handle, int layer, void* stream);
int cf_decoder_layer_finish(int64_t handle, int layer, void* stream);
int cf_decoder_tail(int64_t handle, void* stream);
/* After the caller gathered every shard's (max, idx): pick the winner into the
 * token word and advance seq_len. pairs_val/pairs_idx are device arrays of tp_size. */
int cf_decoder_select_token(int64_t handle, const float* pairs_val, const int* pairs_idx, void* stream);
/* The decoder's device status word (codes as in cf_get_status), read with a blocking 4-byte copy
 * and not cleared.  A loop that already waits for every token (reads it on the host) can poll
 * this cheaply to notice a tensor-parallel peer that stopped answering (7) instead of decoding on
 * with wrong tokens. */
int cf_decoder_status(int64_t handle, int* status);
int cf_decoder_destroy(int64_t handle);

/* -------------------------------------------------------------------------
 * Prompt ingestion.  The reference has no prefill kernel: its end-to-end
 * scripts run the prompt through the HuggingFace model and copy the caches
 * over (tests/benchmark_full.py:195-199, tests/benchmark_decode_6b9.py:40-50).
 * This is the linear layer of that pass as a tensor-core GEMM:
 *   out[m, n] = act(x[m, k] . weight[n, k]^T + bias[n] + residual[m, n])
 * all fp16, fp32 accumulation; bias and residual may be NULL; residual only
 * with CF_ACT_NONE.  n and k must be multiples of 8.  Asynchronous on `stream`.
 * ------------------------------------------------------------------------- */
#define CF_ACT_NONE 0
#define CF_ACT_GELU_TANH 1
#define CF_ACT_GELU_ERF 2
int cf_prefill_linear(const void* x, const void* weight, const void* bias, const void* residual, void* out,
                      int64_t m, int64_t n, int64_t k, int act, void* stream);

/* The rest of a GPT-NeoX block's prompt pass that is not a GEMM or the causal attention, as two kernels.
 * cf_prefill_layernorm2: y1 = LayerNorm(x; gamma1, beta1) and, when y2 != NULL, y2 = LayerNorm(x; gamma2, beta2)
 * for m rows of `hidden` fp16 values in ONE pass over x (the input and post-attention norms of a parallel-residual
 * block see the same x and share mean and variance); fp32 statistics, two-pass, eps as given.
 * cf_prefill_rope_split: qkv [m][heads][3][head_dim] (the fused projection's per-head q, k, v order) ->
 * q_out [m][heads][head_dim] with rotate-half RoPE on the first `rotary` dims, the rotated keys into
 * k_rows[i * kv_row_stride ...] and the values into v_rows[i * kv_row_stride ...] (the caches' first m rows);
 * row i is position i; cos / sin are [m][rotary] fp32.  Same arithmetic as the decode kernel's, so a cache filled
 * here matches one filled token by token.  Asynchronous on `stream`. */
int cf_prefill_layernorm2(const void* x, const void* gamma1, const void* beta1, const void* gamma2, const void* beta2,
                          void* y1, void* y2, int64_t m, int64_t hidden, float eps, void* stream);
int cf_prefill_rope_split(const void* qkv, const float* cos, const float* sin, void* q_out, void* k_rows, void* v_rows,
                          int64_t m, int64_t heads, int64_t head_dim, int64_t rotary, int64_t kv_row_stride, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* CLUSTERFUSION_B200_H_ */
