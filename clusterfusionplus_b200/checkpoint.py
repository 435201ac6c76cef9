"""HuggingFace GPT-NeoX (Pythia) checkpoints -> the fused fp16 layout this library decodes from.

The reference pulls the twelve per-layer tensors out of a loaded
`GPTNeoXForCausalLM` by attribute (tests/benchmark_decode_6b9.py:56-72 of the
reference); this module does the same from a state dict, so a checkpoint can be
converted without instantiating the model, and derives the geometry and the
activation flavour from the HF config.

HF's `query_key_value` rows are already interleaved per head as [Q_h; K_h; V_h]
(GPTNeoXAttention views the projection as [..., heads, 3 * head_dim]), which is the
row order CfLayerWeights.qkv_weight wants: conversion is renaming, casting and
moving to the device.
"""
from __future__ import annotations

from typing import Dict, List, Mapping, Sequence, Tuple

import torch

from ._lib import CF_DECODER_GELU_ERF, CfDims

# HF sub-module name -> key of the per-layer dict (CfLayerWeights field)
_LAYER_MAP = {
    "input_layernorm.weight": "ln_weight", "input_layernorm.bias": "ln_bias",
    "post_attention_layernorm.weight": "post_ln_weight", "post_attention_layernorm.bias": "post_ln_bias",
    "attention.query_key_value.weight": "qkv_weight", "attention.query_key_value.bias": "qkv_bias",
    "attention.dense.weight": "o_weight", "attention.dense.bias": "o_bias",
    "mlp.dense_h_to_4h.weight": "mlp_up_weight", "mlp.dense_h_to_4h.bias": "mlp_up_bias",
    "mlp.dense_4h_to_h.weight": "mlp_down_weight", "mlp.dense_4h_to_h.bias": "mlp_down_bias",
}
_TANH_ACTS = ("gelu_pytorch_tanh", "gelu_new", "gelu_fast")


def _rope_base(cfg) -> float:
    rp = getattr(cfg, "rope_parameters", None)
    if isinstance(rp, Mapping) and "rope_theta" in rp:
        return float(rp["rope_theta"])
    for name in ("rotary_emb_base", "rope_theta"):
        if getattr(cfg, name, None) is not None:
            return float(getattr(cfg, name))
    return 10000.0


def _rotary_pct(cfg) -> float:
    rp = getattr(cfg, "rope_parameters", None)
    if isinstance(rp, Mapping) and "partial_rotary_factor" in rp:
        return float(rp["partial_rotary_factor"])
    for name in ("rotary_pct", "partial_rotary_factor"):
        if getattr(cfg, name, None) is not None:
            return float(getattr(cfg, name))
    return 1.0


def describe_config(cfg) -> Tuple[CfDims, int, float]:
    """(geometry, CF_DECODER_* flags, rope base) of an HF GPTNeoXConfig; raises
    RuntimeError for variants the fused layer does not compute."""
    H, NH = int(cfg.hidden_size), int(cfg.num_attention_heads)
    if H % NH:
        raise RuntimeError(f"hidden_size {H} is not a multiple of num_attention_heads {NH}")
    if not getattr(cfg, "use_parallel_residual", True):
        raise RuntimeError("only the parallel-residual GPT-NeoX block is fused (use_parallel_residual=True)")
    if abs(float(getattr(cfg, "layer_norm_eps", 1e-5)) - 1e-5) > 1e-12:
        raise RuntimeError("LayerNorm epsilon other than 1e-5 is not supported")
    for name in ("rope_parameters", "rope_scaling"):
        rs = getattr(cfg, name, None)
        kind = (rs.get("rope_type") or rs.get("type")) if isinstance(rs, Mapping) else None
        if kind not in (None, "default"):
            raise RuntimeError(f"rope scaling {kind!r} is not supported")
    act = getattr(cfg, "hidden_act", "gelu")
    if act == "gelu":
        flags = CF_DECODER_GELU_ERF
    elif act in _TANH_ACTS:
        flags = 0
    else:
        raise RuntimeError(f"hidden_act {act!r} is not supported (gelu or a tanh GELU)")
    d = CfDims()
    d.hidden, d.heads, d.head_dim = H, NH, H // NH
    d.rotary = int(d.head_dim * _rotary_pct(cfg))
    d.ffn, d.vocab = int(cfg.intermediate_size), int(cfg.vocab_size)
    return d, flags, _rope_base(cfg)


def convert_state_dict(sd: Mapping[str, torch.Tensor], cfg, device="cuda",
                       dtype=torch.float16) -> Tuple[List[Dict[str, torch.Tensor]], Dict[str, torch.Tensor]]:
    """(layers, head) in the layout PythiaDecoder takes, from the state dict of an HF
    `GPTNeoXForCausalLM`.  Missing biases (attention_bias=False) become zeros; a tied
    LM head reuses the embedding."""
    d, _, _ = describe_config(cfg)

    def put(t: torch.Tensor) -> torch.Tensor:
        return t.detach().to(device=device, dtype=dtype).contiguous()

    prefix = "gpt_neox." if any(k.startswith("gpt_neox.") for k in sd) else ""
    sizes = {"qkv_bias": 3 * d.hidden, "o_bias": d.hidden, "mlp_up_bias": d.ffn, "mlp_down_bias": d.hidden}
    layers = []
    for i in range(int(cfg.num_hidden_layers)):
        w = {}
        for src, dst in _LAYER_MAP.items():
            key = f"{prefix}layers.{i}.{src}"
            if key in sd:
                w[dst] = put(sd[key])
            elif dst in sizes:
                w[dst] = torch.zeros(sizes[dst], device=device, dtype=dtype)
            else:
                raise RuntimeError(f"state dict has no {key}")
        if w["qkv_weight"].shape != (3 * d.hidden, d.hidden) or w["mlp_up_weight"].shape != (d.ffn, d.hidden):
            raise RuntimeError(f"layer {i}: tensor shapes do not match the config")
        layers.append(w)
    embed = put(sd[f"{prefix}embed_in.weight"])
    out_key = "embed_out.weight"
    head = {
        "embed_in": embed,
        "final_ln_weight": put(sd[f"{prefix}final_layer_norm.weight"]),
        "final_ln_bias": put(sd[f"{prefix}final_layer_norm.bias"]),
        "embed_out": put(sd[out_key]) if out_key in sd else embed,
    }
    return layers, head


def load_decoder(sd: Mapping[str, torch.Tensor], cfg, max_seq: int, device="cuda", use_graph: bool = True):
    """A PythiaDecoder over freshly allocated KV caches for an HF GPT-NeoX checkpoint."""
    from .decoder import PythiaDecoder

    d, flags, base = describe_config(cfg)
    if d.vocab % 8:
        raise RuntimeError(f"vocab_size {d.vocab} must be a multiple of 8")
    layers, head = convert_state_dict(sd, cfg, device)
    kvw = d.heads * d.head_dim
    caches = [(torch.zeros(max_seq, kvw, device=device, dtype=torch.float16),
               torch.zeros(max_seq, kvw, device=device, dtype=torch.float16)) for _ in layers]
    return PythiaDecoder(d, layers, head, caches, max_seq, use_graph=use_graph, flags=flags, rope_base=base)
