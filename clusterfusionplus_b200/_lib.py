"""ctypes binding of libclusterfusion_b200.so (declared in include/clusterfusion_b200.h).

The library is the product: there is no Python or CPU implementation behind
these calls.  If the shared object is missing, importing this module raises.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
# CLUSTERFUSION_B200_LIB names another build of the same library (A/B comparisons of kernel variants)
LIB_PATH = os.environ.get("CLUSTERFUSION_B200_LIB") or os.path.join(_HERE, "lib", "libclusterfusion_b200.so")

CF_PYTHIA_2B8 = 0
CF_PYTHIA_6B9 = 1


class CfDims(C.Structure):
    _fields_ = [("hidden", C.c_int), ("heads", C.c_int), ("head_dim", C.c_int), ("rotary", C.c_int),
                ("ffn", C.c_int), ("vocab", C.c_int)]


class CfLayerWeights(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "qkv_weight", "qkv_bias", "o_weight", "o_bias", "ln_weight", "ln_bias", "post_ln_weight",
        "post_ln_bias", "mlp_up_weight", "mlp_up_bias", "mlp_down_weight", "mlp_down_bias")]


class CfLayerIO(C.Structure):
    _fields_ = [("input", C.c_void_p), ("k_cache", C.c_void_p), ("v_cache", C.c_void_p),
                ("kv_rows", C.c_int64), ("cos", C.c_void_p), ("sin", C.c_void_p), ("output", C.c_void_p),
                ("k_new", C.c_void_p), ("v_new", C.c_void_p), ("attn_output", C.c_void_p),
                ("mlp_intermediate", C.c_void_p)]


class CfStepArgs(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in (
        "input", "ln_weight", "ln_bias", "qkv_bias", "o_bias", "cos", "sin", "k_cache", "v_cache",
        "post_ln_weight", "post_ln_bias", "mlp_up_bias", "mlp_down_bias")]


class CfDecoderConfig(C.Structure):
    _fields_ = [("dims", CfDims), ("n_layers", C.c_int), ("max_seq_len", C.c_int64), ("tp_size", C.c_int),
                ("tp_rank", C.c_int), ("cos_table", C.c_void_p), ("sin_table", C.c_void_p), ("flags", C.c_int)]


CF_DECODER_GELU_ERF = 1
CF_ACT_NONE, CF_ACT_GELU_TANH, CF_ACT_GELU_ERF = 0, 1, 2


class CfHeadWeights(C.Structure):
    _fields_ = [("embed_in", C.c_void_p), ("final_ln_weight", C.c_void_p), ("final_ln_bias", C.c_void_p),
                ("embed_out", C.c_void_p), ("vocab_offset", C.c_int)]


# every symbol include/clusterfusion_b200.h declares: (restype, argtypes)
_P = C.POINTER
SIGNATURES = {
    "cf_last_error": (C.c_char_p, []),
    "cf_model_dims": (C.c_int, [C.c_int, _P(CfDims)]),
    "cf_launch_info": (C.c_int, [C.c_int] + [_P(C.c_int)] * 5),
    "cf_get_status": (C.c_int, [_P(C.c_int)]),
    "cf_pythia_decoder_layer": (C.c_int, [C.c_int, _P(CfLayerWeights), _P(CfLayerIO), C.c_int64, C.c_void_p]),
    "cf_pythia_decoder_layer_split": (C.c_int, [C.c_int, _P(CfLayerWeights), _P(CfLayerIO), C.c_int64, C.c_void_p]),
    "cf_pythia_decoder_layer_noalloc": (C.c_int, [C.c_int, _P(CfLayerWeights), _P(CfLayerIO), C.c_int64, C.c_void_p]),
    "cf_llama_decoder_layer_sglang": (C.c_int, [C.c_void_p] * 6 + [C.c_int64, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p]
                                      + [C.c_void_p] * 5),
    "cf_llama_decoder_layer_batch_sglang": (C.c_int, [C.c_void_p] * 10 + [C.c_int, C.c_void_p, C.c_float, C.c_void_p, C.c_void_p,
                                                       C.c_int64, C.c_void_p]),
    "cf_llama_mlp_batch_sglang": (C.c_int, [C.c_void_p] * 5 + [C.c_float, C.c_int64, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "cf_llama_mlp_sglang": (C.c_int, [C.c_void_p] * 5 + [C.c_float, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "cf_batch_begin": (C.c_int, []),
    "cf_batch_end": (C.c_int, [C.c_void_p]),
    "cf_batch_abort": (C.c_int, []),
    "cf_debug_run_phases": (C.c_int, [C.c_int, _P(CfLayerWeights), _P(CfLayerIO), C.c_int64, C.c_int, C.c_void_p]),
    "cf_debug_set_trace": (C.c_int, [C.c_void_p, C.c_int64]),
    "cf_debug_set_llama_batch_trace": (C.c_int, [C.c_void_p, C.c_int64]),
    "cf_debug_stream_rows": (C.c_int, [C.c_void_p, C.c_int64, C.c_int64, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p]),
    "cf_pythia_attention_only": (C.c_int, [C.c_int, _P(CfLayerWeights), _P(CfLayerIO), C.c_int64, C.c_void_p]),
    "cf_pythia_mlp_only": (C.c_int, [C.c_int] + [C.c_void_p] * 7),
    "cf_pythia_create_graph_context": (C.c_int, [C.c_int, C.c_int64] + [C.c_void_p] * 6 + [C.c_int64]),
    "cf_pythia_graph_decode_step": (C.c_int, [C.c_int, C.c_int64, _P(CfStepArgs), C.c_int64, C.c_void_p,
                                              _P(C.c_void_p), _P(C.c_void_p), _P(C.c_void_p)]),
    "cf_pythia_graph_set_device_state": (C.c_int, [C.c_int, C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64]),
    "cf_pythia_destroy_graph_context": (C.c_int, [C.c_int, C.c_int64]),
    "cf_decoder_create": (C.c_int, [_P(CfDecoderConfig), _P(C.c_int64)]),
    "cf_decoder_set_layer": (C.c_int, [C.c_int64, C.c_int, _P(CfLayerWeights), C.c_void_p, C.c_void_p]),
    "cf_decoder_set_head": (C.c_int, [C.c_int64, _P(CfHeadWeights)]),
    "cf_decoder_finalize": (C.c_int, [C.c_int64]),
    "cf_decoder_state": (C.c_int, [C.c_int64] + [_P(C.c_void_p)] * 7),
    "cf_decoder_tp_export": (C.c_int, [C.c_int64, C.c_void_p]),
    "cf_decoder_tp_connect": (C.c_int, [C.c_int64, C.c_void_p]),
    "cf_decoder_tp_buffer": (C.c_int, [C.c_int64, _P(C.c_void_p), _P(C.c_int64)]),
    "cf_decoder_tp_connect_pointers": (C.c_int, [C.c_int64, _P(C.c_void_p)]),
    "cf_decoder_step": (C.c_int, [C.c_int64, C.c_void_p]),
    "cf_decoder_layer_partial": (C.c_int, [C.c_int64, C.c_int, C.c_void_p]),
    "cf_decoder_layer_finish": (C.c_int, [C.c_int64, C.c_int, C.c_void_p]),
    "cf_decoder_tail": (C.c_int, [C.c_int64, C.c_void_p]),
    "cf_decoder_select_token": (C.c_int, [C.c_int64, C.c_void_p, C.c_void_p, C.c_void_p]),
    "cf_decoder_destroy": (C.c_int, [C.c_int64]),
    "cf_decoder_status": (C.c_int, [C.c_int64, _P(C.c_int)]),
    "cf_debug_noalloc_scratch": (C.c_int, [_P(C.c_void_p), _P(C.c_int64), _P(C.c_int64)]),
    "cf_prefill_linear": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64,
                                    C.c_int64, C.c_int, C.c_void_p]),
    "cf_prefill_layernorm2": (C.c_int, [C.c_void_p] * 7 + [C.c_int64, C.c_int64, C.c_float, C.c_void_p]),
    "cf_prefill_rope_split": (C.c_int, [C.c_void_p] * 6 + [C.c_int64] * 5 + [C.c_void_p]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python clusterfusionplus_b200/build.py` "
            "(nvcc, sm_100a). There is no fallback implementation.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    msg = lib.cf_last_error()
    return msg.decode() if msg else ""


def check(rc: int) -> None:
    """Raise RuntimeError (the exception type the reference's binding raises) on failure."""
    if rc != 0:
        raise RuntimeError(f"clusterfusion_b200: {last_error()} (code {rc})")
