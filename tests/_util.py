"""Shared helpers of the GPU parity tests (all calls go through the ctypes C ABI
behind the `clusterfusion` operator functions)."""
import torch

from oracle import pythia_oracle as O

# parity bar of this path: output hidden state and new K/V against the fp32 oracle
MAX_ABS = 2e-2
REL_L2 = 1e-3

ARG_ORDER = ("qkv_weight", "qkv_bias", "o_weight", "o_bias")


def layer_args(x, w, k, v, cos, sin, seq):
    """Positional argument list of pythia_*_decoder_layer (include/pybind.cpp:109-129)."""
    return [x, w["qkv_weight"], w["qkv_bias"], w["o_weight"], w["o_bias"], k, v, w["ln_weight"], w["ln_bias"],
            cos, sin, w["post_ln_weight"], w["post_ln_bias"], w["mlp_up_weight"], w["mlp_up_bias"],
            w["mlp_down_weight"], w["mlp_down_bias"], seq]


def step_args(ctx_id, x, w, k, v, cos, sin, seq):
    """Positional argument list of pythia_*_graph_decode_step (include/pybind.cpp:217-233)."""
    return [ctx_id, x, w["ln_weight"], w["ln_bias"], w["qkv_bias"], w["o_bias"], cos, sin, k, v,
            w["post_ln_weight"], w["post_ln_bias"], w["mlp_up_bias"], w["mlp_down_bias"], seq]


def make_case(model, seq, rows=None, wseed=1234, xseed=7, device="cuda:0", std=0.02):
    s = O.SHAPES[model]
    rows = rows or seq + 3
    w = O.make_layer_weights(s, 0, seed=wseed, device=device, std=std)
    x = O.seeded_normal((1, s.hidden), xseed, device=device)
    k, v = O.make_kv_cache(s, seq, rows, xseed + 100, device=device)
    cos, sin = O.rope_table(rows, s.rotary, device=device)
    return s, w, x, k, v, cos[seq].contiguous(), sin[seq].contiguous()


def assert_close(got, ref, what):
    mx, rl = O.compare(got, ref)
    assert mx <= MAX_ABS and rl <= REL_L2, f"{what}: max-abs {mx:.3e} (<= {MAX_ABS}), rel-L2 {rl:.3e} (<= {REL_L2})"
    return mx, rl
