"""Whole-model greedy decode on one GPU: the decode loop the reference drives from
Python (tests/benchmark_decode_6b9.py:133-198: embed_in -> 32 layer ops ->
final LayerNorm -> embed_out -> argmax -> .item()) as ONE persistent launch per
token, optionally captured in a CUDA graph.  Token id and sequence length live
in device memory, so the same graph replays for every token.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import _lib
from ._lib import CF_ACT_GELU_ERF, CF_ACT_GELU_TANH, CF_ACT_NONE, CF_DECODER_GELU_ERF, CfDecoderConfig, CfDims, CfHeadWeights, CfLayerWeights, check, lib
from .api import _req, _wrap

_LAYER_KEYS = {
    "qkv_weight": "qkv_weight", "qkv_bias": "qkv_bias", "o_weight": "o_weight", "o_bias": "o_bias",
    "ln_weight": "ln_weight", "ln_bias": "ln_bias", "post_ln_weight": "post_ln_weight",
    "post_ln_bias": "post_ln_bias", "mlp_up_weight": "mlp_up_weight", "mlp_up_bias": "mlp_up_bias",
    "mlp_down_weight": "mlp_down_weight", "mlp_down_bias": "mlp_down_bias",
}


def rope_table(max_pos: int, rotary: int, device, base: float = 10000.0):
    """[max_pos, rotary] fp32 cos/sin with emb = cat(freqs, freqs)
    (precompute_rope_embeddings, tests/benchmark_decode_6b9.py:23-34 of the reference)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary, 2, dtype=torch.float32, device=device) / rotary))
    pos = torch.arange(0, max_pos, dtype=torch.float32, device=device)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().contiguous(), emb.sin().contiguous()


def layer_weights_struct(d: CfDims, w: Dict[str, torch.Tensor]) -> CfLayerWeights:
    H, KVW, F = d.hidden, d.heads * d.head_dim, d.ffn
    sizes = {"qkv_weight": 3 * KVW * H, "qkv_bias": 3 * KVW, "o_weight": H * KVW, "o_bias": H, "ln_weight": H,
             "ln_bias": H, "post_ln_weight": H, "post_ln_bias": H, "mlp_up_weight": F * H, "mlp_up_bias": F,
             "mlp_down_weight": H * F, "mlp_down_bias": H}
    s = CfLayerWeights()
    for field, key in _LAYER_KEYS.items():
        setattr(s, field, _req(w[key], key, sizes[field]))
    return s


def prefill_linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
                   residual: Optional[torch.Tensor] = None, act: int = CF_ACT_NONE) -> torch.Tensor:
    """act(x @ weight.T + bias + residual) for fp16 x [m, k], weight [n, k] on the tensor cores
    (cf_prefill_linear: TMA-fed tcgen05 GEMM with the bias, GELU and residual fused in)."""
    m, k = x.shape
    n = weight.shape[0]
    out = torch.empty(m, n, device=x.device, dtype=torch.float16)
    check(lib.cf_prefill_linear(_req(x, "x", m * k), _req(weight, "weight", n * k),
                                None if bias is None else _req(bias, "bias", n),
                                None if residual is None else _req(residual, "residual", m * n),
                                out.data_ptr(), m, n, k, act, torch.cuda.current_stream().cuda_stream))
    return out


class PythiaDecoder:
    """Greedy decoder over caller-owned fp16 weights and KV caches.

    layers : list of dicts with the 12 tensors of a layer (keys as in CfLayerWeights)
    head   : dict with embed_in [V,H], final_ln_weight, final_ln_bias, embed_out [V,H]
    caches : list of (k_cache, v_cache), each [max_seq, heads*head_dim] fp16
    """

    def __init__(self, dims: CfDims, layers: Sequence[Dict[str, torch.Tensor]], head: Dict[str, torch.Tensor],
                 caches: Sequence, max_seq: int, use_graph: bool = True, flags: int = 0,
                 rope_base: float = 10000.0):
        self.dims, self.layers, self.head, self.caches = dims, list(layers), head, list(caches)
        self.max_seq = int(max_seq)
        self.flags = int(flags)
        self.device = head["embed_in"].device
        self.cos, self.sin = rope_table(self.max_seq, dims.rotary, self.device, rope_base)
        cfg = CfDecoderConfig()
        cfg.dims = dims
        cfg.n_layers = len(self.layers)
        cfg.max_seq_len = self.max_seq
        cfg.tp_size, cfg.tp_rank = 1, 0
        cfg.cos_table, cfg.sin_table = self.cos.data_ptr(), self.sin.data_ptr()
        cfg.flags = self.flags
        h = C.c_int64(0)
        check(lib.cf_decoder_create(C.byref(cfg), C.byref(h)))
        self.handle = h.value
        KVW = dims.heads * dims.head_dim
        for i, (w, (k, v)) in enumerate(zip(self.layers, self.caches)):
            if k.shape != (self.max_seq, KVW) or v.shape != (self.max_seq, KVW):
                raise RuntimeError(f"layer {i}: caches must be [{self.max_seq}, {KVW}]")
            check(lib.cf_decoder_set_layer(self.handle, i, C.byref(layer_weights_struct(dims, w)),
                                           _req(k, "k_cache", k.numel()), _req(v, "v_cache", v.numel())))
        hw = CfHeadWeights()
        hw.embed_in = _req(head["embed_in"], "embed_in", head["embed_in"].numel())
        hw.final_ln_weight = _req(head["final_ln_weight"], "final_ln_weight", dims.hidden)
        hw.final_ln_bias = _req(head["final_ln_bias"], "final_ln_bias", dims.hidden)
        hw.embed_out = _req(head["embed_out"], "embed_out", dims.vocab * dims.hidden)
        hw.vocab_offset = 0
        check(lib.cf_decoder_set_head(self.handle, C.byref(hw)))
        check(lib.cf_decoder_finalize(self.handle))
        p = [C.c_void_p() for _ in range(7)]
        check(lib.cf_decoder_state(self.handle, *[C.byref(x) for x in p]))
        dev = self.device
        self.token = torch.as_tensor(_IntView(p[0].value, (1,)), device=dev)
        self.seq_len = torch.as_tensor(_IntView(p[1].value, (1,)), device=dev)
        self.logits = torch.as_tensor(_F32View(p[2].value, (dims.vocab,)), device=dev)
        self.hidden = _wrap(p[3].value, (1, dims.hidden), dev)
        self.use_graph = use_graph
        self._graph: Optional[torch.cuda.CUDAGraph] = None

    def reset(self, seq_len: int, token: int) -> None:
        """Position the decoder: `seq_len` rows of every cache are valid, `token` is fed next."""
        self.seq_len.fill_(int(seq_len))
        self.token.fill_(int(token))

    def _enqueue(self) -> None:
        check(lib.cf_decoder_step(self.handle, torch.cuda.current_stream().cuda_stream))

    def capture(self) -> None:
        """Record one token step into a CUDA graph (state words are restored afterwards)."""
        seq0, tok0 = self.seq_len.clone(), self.token.clone()
        # warm-up launch on a side stream, as torch's capture rules want
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            self._enqueue()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._enqueue()
        self._graph = g
        # the warm-up wrote one cache row at seq0 and advanced the state: rewind
        self.seq_len.copy_(seq0)
        self.token.copy_(tok0)

    def step(self) -> None:
        """Decode one token: consumes self.token at position self.seq_len, leaves the
        arg-max token in self.token and seq_len + 1 in self.seq_len.  Asynchronous."""
        if self.use_graph:
            if self._graph is None:
                self.capture()
            self._graph.replay()
        else:
            self._enqueue()

    def generate(self, first_token: int, seq_len: int, n_tokens: int) -> List[int]:
        """Greedy rollout; returns the n_tokens generated ids (one host read per token,
        like the reference loop's .item())."""
        self.reset(seq_len, first_token)
        out = []
        for _ in range(n_tokens):
            self.step()
            out.append(int(self.token.item()))
        return out

    @torch.no_grad()
    def prefill(self, tokens: Sequence[int]) -> None:
        """Ingest a prompt.  Rows [0, n-1) of every cache are computed for all prompt positions
        at once: the four linear layers of a block run as tensor-core GEMMs with their bias,
        GELU and residual fused (cf_prefill_linear), both LayerNorms as one kernel (cf_prefill_layernorm2), RoPE
        and the cache rows as another (cf_prefill_rope_split); the causal attention over the prompt is torch's
        library kernel.  The reference has no prefill of its own and
        leaves it to the HuggingFace model (tests/benchmark_full.py:195-199).  The decoder is
        then positioned on the last prompt token, so the next step() consumes it through the
        fused decode kernel and yields the first generated token."""
        ids = torch.as_tensor(list(tokens), dtype=torch.long, device=self.device)
        n = int(ids.numel())
        if n < 1 or n > self.max_seq - 1:
            raise RuntimeError(f"prompt of {n} tokens does not fit {self.max_seq} cache rows")
        m = n - 1
        if m > 0:
            d = self.dims
            H, NH, D, R = d.hidden, d.heads, d.head_dim, d.rotary
            gelu = CF_ACT_GELU_ERF if (self.flags & CF_DECODER_GELU_ERF) else CF_ACT_GELU_TANH
            st = torch.cuda.current_stream().cuda_stream
            KVW = NH * D
            cos_p, sin_p = _req(self.cos, "cos", m * R, torch.float32, exact=False), _req(self.sin, "sin", m * R, torch.float32, exact=False)
            x = self.head["embed_in"][ids[:m]].contiguous()
            y1, y2 = torch.empty_like(x), torch.empty_like(x)
            q = torch.empty(m, NH, D, device=self.device, dtype=torch.float16)
            for w, (kc, vc) in zip(self.layers, self.caches):
                # both LayerNorms of the block in one pass over x (cf_prefill_layernorm2)
                check(lib.cf_prefill_layernorm2(x.data_ptr(), _req(w["ln_weight"], "ln_weight", H), _req(w["ln_bias"], "ln_bias", H),
                                                _req(w["post_ln_weight"], "post_ln_weight", H),
                                                _req(w["post_ln_bias"], "post_ln_bias", H), y1.data_ptr(), y2.data_ptr(), m, H,
                                                1e-5, st))
                qkv = prefill_linear(y1, w["qkv_weight"], w["qkv_bias"])          # [m, NH, 3, D]
                # rotated queries, rotated keys and values straight into the caches' first m rows (cf_prefill_rope_split)
                check(lib.cf_prefill_rope_split(qkv.data_ptr(), cos_p, sin_p, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), m, NH, D, R,
                                                KVW, st))
                k, v = kc[:m].view(m, NH, D), vc[:m].view(m, NH, D)
                attn = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None],
                                                      v.transpose(0, 1)[None], is_causal=True)
                attn = attn[0].transpose(0, 1).reshape(m, NH * D).contiguous()
                mid = prefill_linear(y2, w["mlp_up_weight"], w["mlp_up_bias"], act=gelu)
                # parallel residual: x + attention branch, then + MLP branch, each add in a GEMM epilogue
                h = prefill_linear(attn, w["o_weight"], w["o_bias"], residual=x)
                x = prefill_linear(mid, w["mlp_down_weight"], w["mlp_down_bias"], residual=h)
        self.reset(m, int(ids[-1].item()))

    def generate_from_prompt(self, tokens: Sequence[int], n_tokens: int) -> List[int]:
        """prefill(tokens), then n_tokens greedy steps; returns the generated ids."""
        self.prefill(tokens)
        out = []
        for _ in range(n_tokens):
            self.step()
            out.append(int(self.token.item()))
        return out

    def close(self) -> None:
        if self.handle:
            self._graph = None
            check(lib.cf_decoder_destroy(self.handle))
            self.handle = 0

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


class _IntView:
    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<i4", "data": (ptr, False),
                                         "version": 3, "strides": None}


class _F32View:
    def __init__(self, ptr, shape):
        self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": "<f4", "data": (ptr, False),
                                         "version": 3, "strides": None}
