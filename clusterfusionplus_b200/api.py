"""Operator API of the reference's `clusterfusion` module for the Pythia decode path.

Same names, positional order and return values as the pybind table of the
reference (include/pybind.cpp:285-297); each function validates its tensors
(the reference validates nothing) and forwards raw pointers to the C ABI on
torch's current stream.  No computation happens in Python.
"""
from __future__ import annotations

import ctypes as C
from typing import Tuple

import torch

from . import _lib
from ._lib import CF_PYTHIA_2B8, CF_PYTHIA_6B9, CfLayerIO, CfLayerWeights, CfStepArgs, check, lib

_DIMS = {}


def model_dims(model: int) -> _lib.CfDims:
    if model not in _DIMS:
        d = _lib.CfDims()
        check(lib.cf_model_dims(model, C.byref(d)))
        _DIMS[model] = d
    return _DIMS[model]


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _req(t: torch.Tensor, name: str, numel: int, dtype=torch.float16, exact: bool = True) -> int:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name}: expected a torch.Tensor")
    if not t.is_cuda:
        raise RuntimeError(f"{name}: expected a CUDA tensor, got {t.device}")
    if t.device.index != torch.cuda.current_device():
        raise RuntimeError(f"{name}: tensor is on {t.device} but the current device is cuda:{torch.cuda.current_device()}")
    if t.dtype != dtype:
        raise RuntimeError(f"{name}: expected dtype {dtype}, got {t.dtype}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name}: expected a contiguous tensor")
    if (exact and t.numel() != numel) or (not exact and t.numel() < numel):
        raise RuntimeError(f"{name}: expected {'' if exact else 'at least '}{numel} elements, got shape {tuple(t.shape)}")
    if t.data_ptr() % 16 != 0:
        raise RuntimeError(f"{name}: storage must be 16-byte aligned")
    return t.data_ptr()


def _cache(t: torch.Tensor, name: str, width: int) -> Tuple[int, int]:
    if not isinstance(t, torch.Tensor) or t.dim() != 2 or t.shape[1] != width:
        raise RuntimeError(f"{name}: expected a [rows, {width}] tensor")
    ptr = _req(t, name, t.numel())
    return ptr, t.shape[0]


def _weights(d, weight_qkv, bias_qkv, weight_o, bias_o, ln_w, ln_b, pln_w, pln_b, up_w, up_b, down_w, down_b):
    H, KVW, F = d.hidden, d.heads * d.head_dim, d.ffn
    w = CfLayerWeights()
    w.qkv_weight = _req(weight_qkv, "weight_qkv", 3 * KVW * H)
    w.qkv_bias = _req(bias_qkv, "bias_qkv", 3 * KVW)
    w.o_weight = _req(weight_o, "weight_o", H * KVW)
    w.o_bias = _req(bias_o, "bias_o", H)
    w.ln_weight = _req(ln_w, "layernorm_weight", H)
    w.ln_bias = _req(ln_b, "layernorm_bias", H)
    w.post_ln_weight = _req(pln_w, "post_ln_weight", H)
    w.post_ln_bias = _req(pln_b, "post_ln_bias", H)
    w.mlp_up_weight = _req(up_w, "mlp_up_weight", F * H)
    w.mlp_up_bias = _req(up_b, "mlp_up_bias", F)
    if down_w is not None:
        w.mlp_down_weight = _req(down_w, "mlp_down_weight", H * F)
        w.mlp_down_bias = _req(down_b, "mlp_down_bias", H)
    return w


def _layer_call(model, fn, input, weight_qkv, bias_qkv, weight_o, bias_o, k_cache, v_cache, layernorm_weight,
                layernorm_bias, cos, sin, post_ln_weight, post_ln_bias, mlp_up_weight, mlp_up_bias,
                mlp_down_weight, mlp_down_bias, current_seq_len):
    d = model_dims(model)
    H, NH, D = d.hidden, d.heads, d.head_dim
    w = _weights(d, weight_qkv, bias_qkv, weight_o, bias_o, layernorm_weight, layernorm_bias, post_ln_weight,
                 post_ln_bias, mlp_up_weight, mlp_up_bias, mlp_down_weight, mlp_down_bias)
    io = CfLayerIO()
    io.input = _req(input, "input", H)
    io.k_cache, rows_k = _cache(k_cache, "k_cache", NH * D)
    io.v_cache, rows_v = _cache(v_cache, "v_cache", NH * D)
    if rows_k != rows_v:
        raise RuntimeError("k_cache and v_cache must have the same number of rows")
    io.kv_rows = rows_k
    io.cos = _req(cos, "cos", d.rotary, torch.float32, exact=False)
    io.sin = _req(sin, "sin", d.rotary, torch.float32, exact=False)
    opts = dict(dtype=torch.float16, device=input.device)
    out = torch.empty((1, H), **opts)
    k = torch.empty((1, NH, D), **opts)
    v = torch.empty((1, NH, D), **opts)
    io.output, io.k_new, io.v_new = out.data_ptr(), k.data_ptr(), v.data_ptr()
    check(fn(model, C.byref(w), C.byref(io), int(current_seq_len), _stream()))
    return out, k, v


def pythia_2b8_decoder_layer(*args):
    """(output[1,2560], k_new[1,32,80], v_new[1,32,80]); writes row current_seq_len of both caches.
    Reference: pythia_2b8_decoder_layer_sm120, include/pybind.cpp:109-129,285."""
    return _layer_call(CF_PYTHIA_2B8, lib.cf_pythia_decoder_layer, *args)


def pythia_6b9_decoder_layer(*args):
    """(output[1,4096], k_new[1,32,128], v_new[1,32,128]); writes row current_seq_len of both caches.
    Reference: pythia_6b9_decoder_layer_sm120, include/pybind.cpp:198-218,294."""
    return _layer_call(CF_PYTHIA_6B9, lib.cf_pythia_decoder_layer, *args)


def pythia_2b8_decoder_layer_split(*args):
    """Two launches, same bits as pythia_2b8_decoder_layer.
    Reference: pythia_2b8_decoder_layer_split_sm120, include/pybind.cpp:132-151,286."""
    return _layer_call(CF_PYTHIA_2B8, lib.cf_pythia_decoder_layer_split, *args)


def pythia_6b9_decoder_layer_split(*args):
    """Split launch for the 6.9B shapes (the reference only ships the 2.8B one)."""
    return _layer_call(CF_PYTHIA_6B9, lib.cf_pythia_decoder_layer_split, *args)


def pythia_2b8_attention_only(input, weight_qkv, bias_qkv, weight_o, bias_o, k_cache, v_cache, layernorm_weight,
                              layernorm_bias, cos, sin, post_ln_weight, post_ln_bias, mlp_up_weight, mlp_up_bias,
                              current_seq_len):
    """(attn_output[1,H], mlp_intermediate[F], k_new, v_new).
    Reference: pythia_2b8_attention_only_sm120, include/pybind.cpp:154-171,287."""
    model = CF_PYTHIA_2B8
    d = model_dims(model)
    H, NH, D = d.hidden, d.heads, d.head_dim
    w = _weights(d, weight_qkv, bias_qkv, weight_o, bias_o, layernorm_weight, layernorm_bias, post_ln_weight,
                 post_ln_bias, mlp_up_weight, mlp_up_bias, None, None)
    io = CfLayerIO()
    io.input = _req(input, "input", H)
    io.k_cache, rows_k = _cache(k_cache, "k_cache", NH * D)
    io.v_cache, rows_v = _cache(v_cache, "v_cache", NH * D)
    if rows_k != rows_v:
        raise RuntimeError("k_cache and v_cache must have the same number of rows")
    io.kv_rows = rows_k
    io.cos = _req(cos, "cos", d.rotary, torch.float32, exact=False)
    io.sin = _req(sin, "sin", d.rotary, torch.float32, exact=False)
    opts = dict(dtype=torch.float16, device=input.device)
    attn = torch.empty((1, H), **opts)
    mid = torch.empty((d.ffn,), **opts)
    k = torch.empty((1, NH, D), **opts)
    v = torch.empty((1, NH, D), **opts)
    io.attn_output, io.mlp_intermediate = attn.data_ptr(), mid.data_ptr()
    io.k_new, io.v_new = k.data_ptr(), v.data_ptr()
    check(lib.cf_pythia_attention_only(model, C.byref(w), C.byref(io), int(current_seq_len), _stream()))
    return attn, mid, k, v


def pythia_2b8_mlp_only(input, attn_output, mlp_intermediate, mlp_down_weight, mlp_down_bias):
    """output[1,H] = input + attn_output + down(mlp_intermediate) + bias.
    Reference: pythia_2b8_mlp_only_sm120, include/pybind.cpp:174-180,288."""
    model = CF_PYTHIA_2B8
    d = model_dims(model)
    H, F = d.hidden, d.ffn
    out = torch.empty((1, H), dtype=torch.float16, device=input.device)
    check(lib.cf_pythia_mlp_only(
        model, _req(input, "input", H), _req(attn_output, "attn_output", H),
        _req(mlp_intermediate, "mlp_intermediate", F), _req(mlp_down_weight, "mlp_down_weight", H * F),
        _req(mlp_down_bias, "mlp_down_bias", H), out.data_ptr(), _stream()))
    return out


def llama_decoder_layer(input, weight_qkv, weight_o, k_cache, v_cache, rms_input_weight, cos, sin):
    """Refused: the reference's first Llama entry point (include/pybind.cpp:66-74,
    include/5090/llama/llama_kernel_dispatch.cu:4-120) takes the projection weights TRANSPOSED (its caller,
    chat/llama/model.py:316-323, stacks wq.T, wk.T, wv.T and passes wo.T), a layout that exists for that
    kernel's TMA boxes.  The same block over weights in nn.Linear layout is llama_decoder_layer_sglang; a
    second set of tensor maps for the transposed layout is not built."""
    raise NotImplementedError(
        "llama_decoder_layer (transposed weights) is not provided; call llama_decoder_layer_sglang with the q/k/v and "
        "output projection weights in nn.Linear layout [out, in] (transpose each block back once, outside the decode loop)")


def llama_decoder_layer_sglang(input, residual, weight_qkv, weight_o, k_cache, v_cache, rms_input_weight, eps, cos, sin):
    """(output[1,4096], residual[1,4096], k_new[1,32,128], v_new[1,32,128]) of the Llama-2-7B attention block.
    `residual` is updated in place to input + residual (fused add + RMSNorm convention) and returned; the
    caches hold exactly the sequence (k_cache.size(0) rows) and are not written.
    Reference: llama_decoder_layer_sglang_sm120, include/pybind.cpp:75-86,281; tests/test_llama.py:149-160."""
    H, NH, D = 4096, 32, 128
    kp, rows_k = _cache(k_cache, "k_cache", H)
    vp, rows_v = _cache(v_cache, "v_cache", H)
    if rows_k != rows_v:
        raise RuntimeError("k_cache and v_cache must have the same number of rows")
    opts = dict(dtype=torch.float16, device=input.device)
    out = torch.empty((1, H), **opts)
    res_out = torch.empty((1, H), **opts)
    k = torch.empty((1, NH, D), **opts)
    v = torch.empty((1, NH, D), **opts)
    check(lib.cf_llama_decoder_layer_sglang(
        _req(input, "input", H), _req(residual, "residual", H), _req(weight_qkv, "weight_qkv", 3 * H * H),
        _req(weight_o, "weight_o", H * H), kp, vp, rows_k, _req(rms_input_weight, "rms_input_weight", H), float(eps),
        _req(cos, "cos", D, torch.float32, exact=False), _req(sin, "sin", D, torch.float32, exact=False),
        out.data_ptr(), res_out.data_ptr(), k.data_ptr(), v.data_ptr(), _stream()))
    residual.copy_(res_out.view_as(residual))
    return out, residual, k, v


def llama_mlp_sglang(input, residual, gate_up_weight, down_weight, rms_weight, eps):
    """(output[1,4096], residual[1,4096]) of the SwiGLU MLP block of a Llama-2-7B layer, same conventions as
    llama_decoder_layer_sglang: `residual` becomes input + residual in place, output =
    down(silu(gate(y)) * up(y)) with y = RMSNorm(residual).  gate_up_weight is [2*ffn, 4096] (gate rows
    first), down_weight [4096, ffn].  The reference leaves this block to the caller
    (tests/test_llama.py:108-110)."""
    H = 4096
    ffn = int(down_weight.shape[-1])
    opts = dict(dtype=torch.float16, device=input.device)
    out = torch.empty((1, H), **opts)
    res_out = torch.empty((1, H), **opts)
    check(lib.cf_llama_mlp_sglang(
        _req(input, "input", H), _req(residual, "residual", H), _req(gate_up_weight, "gate_up_weight", 2 * ffn * H),
        _req(down_weight, "down_weight", H * ffn), _req(rms_weight, "rms_weight", H), float(eps), ffn,
        out.data_ptr(), res_out.data_ptr(), _stream()))
    residual.copy_(res_out.view_as(residual))
    return out, residual


def llama_decoder_layer_batch_decode_sglang(output, residual_output, input, residual, weight_qkv, weight_o,
                                            paged_kv_indptr, paged_kv_indices, k_cache_ptrs, v_cache_ptrs, layer_id,
                                            rms_input_weight, eps, positions, cos_sin):
    """The Llama-2-7B attention block for a batch of decode sequences over a paged KV pool; writes into
    `output` and `residual_output` ([batch, 4096] fp16 each) and returns None, like the reference.
    input / residual [batch, 4096] fp16; paged_kv_indptr [batch + 1] and paged_kv_indices int32 (one pool row per
    token; a sequence's last entry is the slot the new key / value go to); k_cache_ptrs / v_cache_ptrs: int64 /
    uint64 device tensors with one pool pointer per layer ([pool_rows, 4096] fp16 pools); positions [batch] int64;
    cos_sin [max_position, 128] fp32 (64 cosines, 64 sines per row).
    Reference: llama_decoder_layer_batch_sglang_sm120, include/pybind.cpp:90-106,282."""
    H = 4096
    if input.dim() != 2 or input.shape[1] != H:
        raise RuntimeError(f"input: expected [batch, {H}], got {tuple(input.shape)}")
    B = int(input.shape[0])

    def ptrs(t, name):
        if t.dtype not in (torch.int64, torch.uint64):
            raise RuntimeError(f"{name}: expected an int64 / uint64 tensor of device pointers, got {t.dtype}")
        if int(layer_id) < 0 or int(layer_id) >= t.numel():
            raise RuntimeError(f"layer_id {layer_id} outside {name} ({t.numel()} entries)")
        return _req(t, name, t.numel(), t.dtype)

    if paged_kv_indptr.numel() != B + 1:
        raise RuntimeError(f"paged_kv_indptr: expected {B + 1} entries, got {paged_kv_indptr.numel()}")
    if cos_sin.dim() != 2 or cos_sin.shape[1] != 128:
        raise RuntimeError(f"cos_sin: expected [positions, 128] fp32, got {tuple(cos_sin.shape)}")
    check(lib.cf_llama_decoder_layer_batch_sglang(
        _req(output, "output", B * H), _req(residual_output, "residual_output", B * H), _req(input, "input", B * H),
        _req(residual, "residual", B * H), _req(weight_qkv, "weight_qkv", 3 * H * H), _req(weight_o, "weight_o", H * H),
        _req(paged_kv_indptr, "paged_kv_indptr", B + 1, torch.int32),
        _req(paged_kv_indices, "paged_kv_indices", paged_kv_indices.numel(), torch.int32),
        ptrs(k_cache_ptrs, "k_cache_ptrs"), ptrs(v_cache_ptrs, "v_cache_ptrs"), int(layer_id),
        _req(rms_input_weight, "rms_input_weight", H), float(eps), _req(positions, "positions", B, torch.int64),
        _req(cos_sin, "cos_sin", cos_sin.numel(), torch.float32), B, _stream()))
    return None


def llama_mlp_batch_sglang(input, residual, gate_up_weight, down_weight, rms_weight, eps):
    """(output [batch, 4096], residual_out [batch, 4096]) of the SwiGLU MLP block for a batch of rows, weights streamed
    once for all rows (see llama_mlp_sglang for the arithmetic).  `residual` is not modified."""
    H = 4096
    B = int(input.shape[0])
    ffn = int(down_weight.shape[-1])
    opts = dict(dtype=torch.float16, device=input.device)
    out = torch.empty((B, H), **opts)
    res_out = torch.empty((B, H), **opts)
    check(lib.cf_llama_mlp_batch_sglang(
        _req(input, "input", B * H), _req(residual, "residual", B * H), _req(gate_up_weight, "gate_up_weight", 2 * ffn * H),
        _req(down_weight, "down_weight", H * ffn), _req(rms_weight, "rms_weight", H), float(eps), ffn, B,
        out.data_ptr(), res_out.data_ptr(), _stream()))
    return out, res_out


# ---------------------------------------------------------------------------- contexts
class _DeviceView:
    """Zero-copy torch view of a buffer the C library owns."""

    def __init__(self, ptr: int, shape, typestr="<f2"):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False),
                                         "version": 3, "strides": None}


def _wrap(ptr: int, shape, device) -> torch.Tensor:
    return torch.as_tensor(_DeviceView(ptr, shape), device=device)


_ctx_keepalive = {}  # (model, id) -> tensors the context points at
_ctx_views = {}      # (model, id) -> (out, k_new, v_new) views of the static buffers


def _create(model, context_id, k_cache, v_cache, weight_qkv, weight_o, mlp_up_weight, mlp_down_weight, max_seq_len):
    d = model_dims(model)
    H, KVW, F = d.hidden, d.heads * d.head_dim, d.ffn
    kp, rows_k = _cache(k_cache, "k_cache", KVW)
    vp, rows_v = _cache(v_cache, "v_cache", KVW)
    max_seq_len = int(max_seq_len)
    if max_seq_len <= 0 or max_seq_len > min(rows_k, rows_v):
        raise RuntimeError(f"max_seq_len {max_seq_len} exceeds the cache rows ({rows_k}, {rows_v})")
    check(lib.cf_pythia_create_graph_context(
        model, int(context_id), kp, vp, _req(weight_qkv, "weight_qkv", 3 * KVW * H),
        _req(weight_o, "weight_o", H * KVW), _req(mlp_up_weight, "mlp_up_weight", F * H),
        _req(mlp_down_weight, "mlp_down_weight", H * F), max_seq_len))
    key = (model, int(context_id))
    _ctx_keepalive[key] = (k_cache, v_cache, weight_qkv, weight_o, mlp_up_weight, mlp_down_weight)
    _ctx_views.pop(key, None)


def _step(model, context_id, input, layernorm_weight, layernorm_bias, qkv_bias, o_bias, cos, sin, k_cache, v_cache,
          post_ln_weight, post_ln_bias, mlp_up_bias, mlp_down_bias, current_seq_len):
    d = model_dims(model)
    H, NH, D, KVW, F = d.hidden, d.heads, d.head_dim, d.heads * d.head_dim, d.ffn
    a = CfStepArgs()
    a.input = _req(input, "input", H)
    a.ln_weight = _req(layernorm_weight, "layernorm_weight", H)
    a.ln_bias = _req(layernorm_bias, "layernorm_bias", H)
    a.qkv_bias = _req(qkv_bias, "qkv_bias", 3 * KVW)
    a.o_bias = _req(o_bias, "o_bias", H)
    a.cos = _req(cos, "cos", d.rotary, torch.float32, exact=False)
    a.sin = _req(sin, "sin", d.rotary, torch.float32, exact=False)
    a.k_cache, _ = _cache(k_cache, "k_cache", KVW)
    a.v_cache, _ = _cache(v_cache, "v_cache", KVW)
    a.post_ln_weight = _req(post_ln_weight, "post_ln_weight", H)
    a.post_ln_bias = _req(post_ln_bias, "post_ln_bias", H)
    a.mlp_up_bias = _req(mlp_up_bias, "mlp_up_bias", F)
    a.mlp_down_bias = _req(mlp_down_bias, "mlp_down_bias", H)
    po, pk, pv = C.c_void_p(), C.c_void_p(), C.c_void_p()
    check(lib.cf_pythia_graph_decode_step(model, int(context_id), C.byref(a), int(current_seq_len), _stream(),
                                          C.byref(po), C.byref(pk), C.byref(pv)))
    key = (model, int(context_id))
    views = _ctx_views.get(key)
    if views is None:
        dev = input.device
        views = (_wrap(po.value, (1, H), dev), _wrap(pk.value, (1, NH, D), dev), _wrap(pv.value, (1, NH, D), dev))
        _ctx_views[key] = views
    return views


def _destroy(model, context_id):
    check(lib.cf_pythia_destroy_graph_context(model, int(context_id)))
    key = (model, int(context_id))
    _ctx_keepalive.pop(key, None)
    _ctx_views.pop(key, None)


def _set_device_state(model, context_id, seq_len_dev, cos_table, sin_table):
    d = model_dims(model)
    sp = 0 if seq_len_dev is None else _req(seq_len_dev, "seq_len_dev", 1, torch.int32)
    cp = sp_ = 0
    stride = 0
    if cos_table is not None:
        if cos_table.dim() != 2 or cos_table.shape[1] < d.rotary or cos_table.shape != sin_table.shape:
            raise RuntimeError("cos_table / sin_table: expected matching [rows, >= rotary] fp32 tensors")
        cp = _req(cos_table, "cos_table", cos_table.numel(), torch.float32)
        sp_ = _req(sin_table, "sin_table", sin_table.numel(), torch.float32)
        stride = cos_table.shape[1]
    check(lib.cf_pythia_graph_set_device_state(model, int(context_id), sp, cp, sp_, stride))
    _ctx_keepalive[(model, int(context_id), "dev")] = (seq_len_dev, cos_table, sin_table)


def pythia_2b8_create_graph_context(*a):
    """Reference: pythia_2b8_create_graph_context_sm120, include/pybind.cpp:206-215,289."""
    _create(CF_PYTHIA_2B8, *a)


def pythia_2b8_graph_decode_step(*a):
    """Returns views of the context's static buffers (clone to keep).
    Reference: pythia_2b8_graph_decode_step_sm120, include/pybind.cpp:217-233,290."""
    return _step(CF_PYTHIA_2B8, *a)


def pythia_2b8_destroy_graph_context(context_id):
    """Reference: pythia_2b8_destroy_graph_context_sm120, include/pybind.cpp:235,291."""
    _destroy(CF_PYTHIA_2B8, context_id)


def pythia_6b9_create_graph_context(*a):
    """Reference: pythia_6b9_create_graph_context_sm120, include/pybind.cpp:238-247,295."""
    _create(CF_PYTHIA_6B9, *a)


def pythia_6b9_graph_decode_step(*a):
    """Reference: pythia_6b9_graph_decode_step_sm120, include/pybind.cpp:249-265,296."""
    return _step(CF_PYTHIA_6B9, *a)


def pythia_6b9_destroy_graph_context(context_id):
    """Reference: pythia_6b9_destroy_graph_context_sm120, include/pybind.cpp:267,297."""
    _destroy(CF_PYTHIA_6B9, context_id)


def pythia_2b8_graph_set_device_state(context_id, seq_len_dev, cos_table=None, sin_table=None):
    """Extension: let a context read seq_len (int32 tensor) and its RoPE row from device
    memory so a captured CUDA graph of graph_decode_step calls can be replayed."""
    _set_device_state(CF_PYTHIA_2B8, context_id, seq_len_dev, cos_table, sin_table)


def pythia_6b9_graph_set_device_state(context_id, seq_len_dev, cos_table=None, sin_table=None):
    _set_device_state(CF_PYTHIA_6B9, context_id, seq_len_dev, cos_table, sin_table)


def device_status() -> int:
    """Synchronise and return the device status word (0 = every launch completed normally);
    raises RuntimeError if a kernel reported a timeout or a bad sequence length."""
    s = C.c_int(0)
    check(lib.cf_get_status(C.byref(s)))
    return s.value


def launch_info(model: int = CF_PYTHIA_6B9) -> dict:
    v = [C.c_int(0) for _ in range(5)]
    check(lib.cf_launch_info(model, *[C.byref(x) for x in v]))
    return dict(sm_count=v[0].value, grid=v[1].value, cluster=v[2].value, stages=v[3].value, smem_bytes=v[4].value)
