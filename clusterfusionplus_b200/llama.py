"""Llama-2-7B-shaped decoder layers at batch 1: the attention block of the reference
(llama_decoder_layer_sglang, include/pybind.cpp:75-86) followed by the SwiGLU MLP block it leaves
to the caller, chained over a stack of layers without intermediate copies.

The (hidden, residual) pair is handed from block to block the way serving stacks do with a fused
add + RMSNorm: every block first forms residual' = hidden + residual, normalises that, and returns
its own output as the next hidden.  Two buffer pairs ping-pong, so no block reads what it writes.
"""
from __future__ import annotations

from typing import Dict, List, Sequence

import torch

from ._lib import check, lib
from .api import _cache, _req, _stream

H, NH, D = 4096, 32, 128


class LlamaLayerStack:
    """layers: dicts with weight_qkv [3H,H] ([Q;K;V] row blocks), weight_o [H,H], rms_input_weight [H],
    k_cache / v_cache [seq,H] (read-only history), gate_up_weight [2F,H] (gate rows first),
    down_weight [H,F], rms_post_weight [H]."""

    def __init__(self, layers: Sequence[Dict[str, torch.Tensor]], eps: float = 1e-5, one_launch: bool = False):
        self.layers: List[Dict[str, torch.Tensor]] = list(layers)
        self.eps = float(eps)
        # one_launch: the 2 x layers block calls of a step are recorded (cf_batch_begin / cf_batch_end) and run as
        # ONE persistent launch with grid barriers between the blocks, instead of one launch per block.  Same bits;
        # measured slower than the per-block launches replayed from a CUDA graph (3 880 against 3 389 us for 32
        # layers), so it is off unless asked for
        self.one_launch = bool(one_launch)
        dev = self.layers[0]["weight_qkv"].device
        opts = dict(dtype=torch.float16, device=dev)
        self.x = [torch.zeros(1, H, **opts) for _ in range(2)]
        self.r = [torch.zeros(1, H, **opts) for _ in range(2)]
        self.k_new = torch.zeros(len(self.layers), NH, D, **opts)
        self.v_new = torch.zeros(len(self.layers), NH, D, **opts)
        self._args = []
        for i, w in enumerate(self.layers):
            kp, rows = _cache(w["k_cache"], "k_cache", H)
            vp, rows_v = _cache(w["v_cache"], "v_cache", H)
            if rows != rows_v:
                raise RuntimeError(f"layer {i}: k_cache and v_cache must have the same number of rows")
            ffn = int(w["down_weight"].shape[-1])
            self._args.append((
                _req(w["weight_qkv"], "weight_qkv", 3 * H * H), _req(w["weight_o"], "weight_o", H * H), kp, vp, rows,
                _req(w["rms_input_weight"], "rms_input_weight", H),
                _req(w["gate_up_weight"], "gate_up_weight", 2 * ffn * H), _req(w["down_weight"], "down_weight", H * ffn),
                _req(w["rms_post_weight"], "rms_post_weight", H), ffn))

    def step(self, hidden: torch.Tensor, residual: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor):
        """One token through every layer.  Returns (hidden_out, residual_out) as views of internal
        buffers (clone what you keep); the new key / value rows of every layer are in
        self.k_new / self.v_new ([layers, 32, 128]); the caches are not written."""
        st = _stream()
        cp, sp = _req(cos, "cos", D, torch.float32, exact=False), _req(sin, "sin", D, torch.float32, exact=False)
        xa, ra, xb, rb = self.x[0], self.r[0], self.x[1], self.r[1]
        x_in, r_in = _req(hidden, "hidden", H), _req(residual, "residual", H)
        if self.one_launch:
            check(lib.cf_batch_begin())
        try:
            for i, (wqkv, wo, kp, vp, rows, g1, wgu, wd, g2, ffn) in enumerate(self._args):
                check(lib.cf_llama_decoder_layer_sglang(x_in, r_in, wqkv, wo, kp, vp, rows, g1, self.eps, cp, sp,
                                                        xb.data_ptr(), rb.data_ptr(), self.k_new[i].data_ptr(),
                                                        self.v_new[i].data_ptr(), st))
                check(lib.cf_llama_mlp_sglang(xb.data_ptr(), rb.data_ptr(), wgu, wd, g2, self.eps, ffn, xa.data_ptr(),
                                              ra.data_ptr(), st))
                x_in, r_in = xa.data_ptr(), ra.data_ptr()
        except Exception:
            if self.one_launch:
                lib.cf_batch_abort()
            raise
        if self.one_launch:
            check(lib.cf_batch_end(st))
        return xa, ra
