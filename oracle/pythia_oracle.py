"""CPU fp32 oracle for the fused GPT-NeoX/Pythia decoder-layer decode step (batch 1).

TEST INFRASTRUCTURE ONLY.  Nothing in the shipped package imports this module;
it is the checker used by tests/, by ``__graft_entry__.smoke()`` and by the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py``.

What it restates
----------------
The reference checks its kernels against a hand-written torch forward of one
Pythia layer (tests/test_pythia_6b9.py:89-180, tests/test_pythia.py:70-170 in the
reference project) and, end to end, against HuggingFace ``GPTNeoXLayer``
(tests/benchmark_decode_6b9.py:47,227).  This file restates that math in plain
fp32 torch, one function per phase so tests can look at intermediates:

* LayerNorm, biased variance, eps inside the sqrt       (test_pythia_6b9.py:105-111)
* QKV projection, per-head interleaved [Q_h; K_h; V_h]   (test_pythia_6b9.py:116-125)
* partial NeoX rotate-half RoPE on the first R dims      (test_pythia_6b9.py:52-79)
* softmax(q.K^T / sqrt(D)) V over cache rows + new row   (test_pythia_6b9.py:147-160)
* dense, tanh-GELU MLP, parallel residual                (test_pythia_6b9.py:82-86,167-175)
* decode-loop tail: final LayerNorm, untied LM head, argmax
                                                         (benchmark_decode_6b9.py:186-195)

The arithmetic itself lives in third-party code that is not part of the
reference tree: ``transformers`` (GPTNeoXLayer) and ``torch``; the reference pins
no version (setup.py:71).  Pinning: the reference ships no golden vectors for
this path, so the restatement is pinned against the live HuggingFace layer
(transformers 5.5.0 / torch 2.11.0) by ``hf_layer_decode`` below, and small
seeded golden vectors produced by this file are committed under tests/golden/.

Layouts (same as the operator API):
  k_cache, v_cache : [rows >= seq_len+1, NH*D], row = position, head-major columns
  k_new, v_new     : [1, NH, D] (k post-RoPE)
  cos, sin         : fp32 [R] for the current position
"""
from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

LN_EPS = 1e-5
GELU_C = 0.7978845608028654  # sqrt(2/pi)
GELU_K = 0.044715


@dataclass(frozen=True)
class Shape:
    """Model geometry.  Names follow the reference's config.h macros."""
    name: str
    hidden: int      # HIDDEN_DIM
    heads: int       # HEAD_NUM
    head_dim: int    # HEAD_DIM
    rotary: int      # ROTARY_DIM
    ffn: int         # FFN_DIM
    vocab: int
    layers: int = 32


PYTHIA_2B8 = Shape("pythia-2.8b", 2560, 32, 80, 20, 10240, 50304)
PYTHIA_6B9 = Shape("pythia-6.9b", 4096, 32, 128, 32, 16384, 50432)
SHAPES = {"2b8": PYTHIA_2B8, "6b9": PYTHIA_6B9}

# order fixes the per-tensor seed offsets of the generators
LAYER_TENSORS = (
    "ln_weight", "ln_bias", "qkv_weight", "qkv_bias", "o_weight", "o_bias",
    "post_ln_weight", "post_ln_bias", "mlp_up_weight", "mlp_up_bias",
    "mlp_down_weight", "mlp_down_bias",
)


def _tensor_shape(shape: Shape, name: str):
    H, F = shape.hidden, shape.ffn
    return {
        "ln_weight": (H,), "ln_bias": (H,), "post_ln_weight": (H,), "post_ln_bias": (H,),
        "qkv_weight": (3 * H, H), "qkv_bias": (3 * H,),
        "o_weight": (H, H), "o_bias": (H,),
        "mlp_up_weight": (F, H), "mlp_up_bias": (F,),
        "mlp_down_weight": (H, F), "mlp_down_bias": (H,),
    }[name]


def seeded_normal(size, seed: int, mean=0.0, std=1.0, device="cpu") -> torch.Tensor:
    """N(mean, std) drawn in fp32 from a private generator, rounded to fp16."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    t = torch.randn(size, generator=g, dtype=torch.float32, device=device)
    return (t * std + mean).to(torch.float16)


def make_layer_weights(shape: Shape, layer: int, seed: int = 1234, device="cpu",
                       std: float = 0.02) -> Dict[str, torch.Tensor]:
    """Seeded fp16 weights of one layer: linear weights/biases N(0,std), LN gamma
    1+N(0,std), LN beta N(0,std).  Seed = seed + 1000*layer + tensor index."""
    out = {}
    for i, name in enumerate(LAYER_TENSORS):
        mean = 1.0 if name in ("ln_weight", "post_ln_weight") else 0.0
        out[name] = seeded_normal(_tensor_shape(shape, name), seed + 1000 * layer + i,
                                  mean=mean, std=std, device=device)
    return out


def make_head_weights(shape: Shape, seed: int = 1234, device="cpu", std: float = 0.02):
    """Embedding [V,H], final LayerNorm, untied LM head [V,H]."""
    base = seed + 1000 * 1000
    return {
        "embed_in": seeded_normal((shape.vocab, shape.hidden), base + 0, std=std, device=device),
        "final_ln_weight": seeded_normal((shape.hidden,), base + 1, mean=1.0, std=std, device=device),
        "final_ln_bias": seeded_normal((shape.hidden,), base + 2, std=std, device=device),
        "embed_out": seeded_normal((shape.vocab, shape.hidden), base + 3, std=std, device=device),
    }


def make_kv_cache(shape: Shape, seq_len: int, rows: int, seed: int, device="cpu"):
    """Random N(0,1) fp16 history generated head-major [NH, seq, D] (the oracle-side
    layout of the benchmark configs) and laid out as the operator wants it:
    [rows, NH*D] with the first seq_len rows filled and the rest zero."""
    assert rows > seq_len
    NH, D = shape.heads, shape.head_dim
    caches = []
    for j in range(2):
        c = torch.zeros((rows, NH * D), dtype=torch.float16, device=device)
        if seq_len > 0:
            hist = seeded_normal((NH, seq_len, D), seed + j, device=device)
            c[:seq_len] = hist.transpose(0, 1).reshape(seq_len, NH * D)
        caches.append(c)
    return caches[0], caches[1]


def rope_table(max_pos: int, rotary: int, base: float = 10000.0, device="cpu"):
    """cos/sin rows [max_pos, R] fp32, emb = cat(freqs, freqs)
    (benchmark_decode_6b9.py:23-34 of the reference)."""
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary, 2, dtype=torch.float32, device=device) / rotary))
    pos = torch.arange(0, max_pos, dtype=torch.float32, device=device)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().contiguous(), emb.sin().contiguous()


# ----------------------------------------------------------------------------
# phases
# ----------------------------------------------------------------------------

def layer_norm_stats(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    mean = x.mean(dim=-1, keepdim=True)
    var = x.var(dim=-1, keepdim=True, unbiased=False)
    return mean, torch.rsqrt(var + LN_EPS)


def layer_norm(x, gamma, beta):
    mean, rstd = layer_norm_stats(x)
    return (x - mean) * rstd * gamma + beta


def rotate_half(t):
    h = t.shape[-1] // 2
    return torch.cat((-t[..., h:], t[..., :h]), dim=-1)


def rope_partial(t: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rotary: int):
    """t [NH, D]; rotate-half on the first `rotary` dims with cos/sin [rotary]."""
    rot, keep = t[..., :rotary], t[..., rotary:]
    rot = rot * cos + rotate_half(rot) * sin
    return torch.cat([rot, keep], dim=-1)


def gelu_tanh(x):
    return 0.5 * x * (1.0 + torch.tanh(GELU_C * (x + GELU_K * x * x * x)))


def gelu_erf(x):
    return 0.5 * x * (1.0 + torch.erf(x * 0.7071067811865476))


def layer_decode_fp32(shape: Shape, x: torch.Tensor, w: Dict[str, torch.Tensor],
                      k_cache: torch.Tensor, v_cache: torch.Tensor,
                      cos: torch.Tensor, sin: torch.Tensor, seq_len: int,
                      intermediates: Optional[dict] = None, partial: bool = False, act: str = "tanh"):
    """One decode step of one layer in fp32.

    x [1,H]; caches [rows, NH*D] of which rows [0, seq_len) are history (not
    modified here); cos/sin fp32, first R entries used.
    Returns (out [1,H], k_new [1,NH,D], v_new [1,NH,D]) in fp32.

    `shape.heads` / `shape.ffn` may describe a tensor-parallel shard (fewer heads,
    narrower MLP, full hidden width).  With partial=True the result is the shard's
    contribution attn @ Wo^T + mid @ Wdown^T only: no residual, no dense / down bias
    (those are added once, after the partials of all shards are summed).
    act = "tanh" is the reference kernels' GELU (kernel.cuh:39-54), "erf" the exact
    form of the published checkpoints (HF hidden_act "gelu").
    """
    H, NH, D, R = shape.hidden, shape.heads, shape.head_dim, shape.rotary
    f = lambda t: t.detach().to("cpu", torch.float32)
    x = f(x).reshape(1, H)
    cos = f(cos).reshape(-1)[:R]
    sin = f(sin).reshape(-1)[:R]
    W = {k: f(v) for k, v in w.items()}

    y1 = layer_norm(x, W["ln_weight"].reshape(-1), W["ln_bias"].reshape(-1))
    y2 = layer_norm(x, W["post_ln_weight"].reshape(-1), W["post_ln_bias"].reshape(-1))

    qkv = (y1 @ W["qkv_weight"].t() + W["qkv_bias"]).view(NH, 3, D)
    q = rope_partial(qkv[:, 0], cos, sin, R)
    k_new = rope_partial(qkv[:, 1], cos, sin, R)
    v_new = qkv[:, 2]

    k_hist = f(k_cache[:seq_len]).view(seq_len, NH, D)
    v_hist = f(v_cache[:seq_len]).view(seq_len, NH, D)
    k_all = torch.cat([k_hist, k_new[None]], dim=0).transpose(0, 1)  # [NH, S+1, D]
    v_all = torch.cat([v_hist, v_new[None]], dim=0).transpose(0, 1)
    scores = torch.einsum("hd,hsd->hs", q, k_all) / math.sqrt(D)
    p = torch.softmax(scores, dim=-1)
    attn = torch.einsum("hs,hsd->hd", p, v_all).reshape(1, NH * D)

    attn_out = attn @ W["o_weight"].t() + W["o_bias"]
    pre = y2 @ W["mlp_up_weight"].t() + W["mlp_up_bias"]
    mid = gelu_erf(pre) if act == "erf" else gelu_tanh(pre)
    mlp_out = mid @ W["mlp_down_weight"].t() + W["mlp_down_bias"]
    out = x + attn_out + mlp_out
    if partial:
        out = attn @ W["o_weight"].t() + mid @ W["mlp_down_weight"].t()
    if intermediates is not None:
        intermediates.update(y1=y1, y2=y2, q=q, attn=attn, attn_out=attn_out, mid=mid,
                             mlp_out=mlp_out)
    return out, k_new[None].clone(), v_new[None].clone()


def final_logits_fp32(x, head: Dict[str, torch.Tensor]):
    """Decode-loop tail: final LayerNorm then the untied LM head, fp32."""
    f = lambda t: t.detach().to("cpu", torch.float32)
    y = layer_norm(f(x).reshape(1, -1), f(head["final_ln_weight"]), f(head["final_ln_bias"]))
    return y @ f(head["embed_out"]).t()


def round_fp16(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.float16).to(torch.float32)


class OracleModel:
    """Greedy decode of a whole seeded model on CPU in fp32.

    `layers` is a list of per-layer weight dicts (fp16 or fp32), `head` the dict
    of make_head_weights.  Caches are kept in fp32 but every appended row, and
    the hidden state handed from layer to layer, is rounded to fp16 exactly
    where the operator API materialises fp16 tensors (k_new/v_new/cache rows and
    the layer output), so a rollout compares like with like.
    """

    def __init__(self, shape: Shape, layers, head, max_seq: int, round_io: bool = True, act: str = "tanh",
                 rope_base: float = 10000.0):
        self.shape, self.head, self.max_seq, self.round_io, self.act = shape, head, max_seq, round_io, act
        self.layers = [{k: v.detach().to("cpu", torch.float32) for k, v in w.items()} for w in layers]
        W = shape.heads * shape.head_dim
        self.k = [torch.zeros(max_seq, W) for _ in layers]
        self.v = [torch.zeros(max_seq, W) for _ in layers]
        self.cos, self.sin = rope_table(max_seq, shape.rotary, base=rope_base)
        self.seq_len = 0

    def load_cache(self, layer: int, k: torch.Tensor, v: torch.Tensor, seq_len: int):
        self.k[layer][:seq_len] = k[:seq_len].detach().to("cpu", torch.float32)
        self.v[layer][:seq_len] = v[:seq_len].detach().to("cpu", torch.float32)

    def step(self, token: int):
        """Feed one token at position seq_len; returns (logits [V] fp32, hidden [1,H])."""
        s = self.seq_len
        x = self.head["embed_in"][token].detach().to("cpu", torch.float32).reshape(1, -1)
        for i, w in enumerate(self.layers):
            x, kn, vn = layer_decode_fp32(self.shape, x, w, self.k[i], self.v[i],
                                          self.cos[s], self.sin[s], s, act=self.act)
            if self.round_io:
                x, kn, vn = round_fp16(x), round_fp16(kn), round_fp16(vn)
            self.k[i][s] = kn.reshape(-1)
            self.v[i][s] = vn.reshape(-1)
        self.seq_len = s + 1
        return final_logits_fp32(x, self.head).reshape(-1), x


# ----------------------------------------------------------------------------
# pin against HuggingFace GPTNeoXLayer (the oracle named by the reference's
# end-to-end scripts).  Only used by the CPU tests.
# ----------------------------------------------------------------------------

def hf_layer_decode(shape: Shape, x, w, k_cache, v_cache, seq_len: int, position: int):
    """Same decode step through transformers' GPTNeoXLayer in fp32 (eager attention,
    tanh GELU, rotary_pct 0.25, parallel residual).  Returns (out, k_new, v_new)."""
    from transformers import GPTNeoXConfig
    from transformers.cache_utils import DynamicCache
    from transformers.models.gpt_neox.modeling_gpt_neox import GPTNeoXLayer, GPTNeoXRotaryEmbedding

    H, NH, D = shape.hidden, shape.heads, shape.head_dim
    cfg = GPTNeoXConfig(
        hidden_size=H, num_attention_heads=NH, intermediate_size=shape.ffn,
        num_hidden_layers=1, rotary_pct=shape.rotary / D, rotary_emb_base=10000,
        use_parallel_residual=True, layer_norm_eps=LN_EPS, attention_bias=True,
        hidden_act="gelu_pytorch_tanh", max_position_embeddings=max(2048, position + 1),
        hidden_dropout=0.0, attention_dropout=0.0, vocab_size=shape.vocab,
    )
    cfg._attn_implementation = "eager"
    layer = GPTNeoXLayer(cfg, layer_idx=0).float().eval()
    f = lambda t: t.detach().to("cpu", torch.float32)
    sd = {
        "input_layernorm.weight": f(w["ln_weight"]).reshape(-1),
        "input_layernorm.bias": f(w["ln_bias"]).reshape(-1),
        "post_attention_layernorm.weight": f(w["post_ln_weight"]).reshape(-1),
        "post_attention_layernorm.bias": f(w["post_ln_bias"]).reshape(-1),
        "attention.query_key_value.weight": f(w["qkv_weight"]),
        "attention.query_key_value.bias": f(w["qkv_bias"]),
        "attention.dense.weight": f(w["o_weight"]),
        "attention.dense.bias": f(w["o_bias"]),
        "mlp.dense_h_to_4h.weight": f(w["mlp_up_weight"]),
        "mlp.dense_h_to_4h.bias": f(w["mlp_up_bias"]),
        "mlp.dense_4h_to_h.weight": f(w["mlp_down_weight"]),
        "mlp.dense_4h_to_h.bias": f(w["mlp_down_bias"]),
    }
    missing, unexpected = layer.load_state_dict(sd, strict=False)
    assert not unexpected, unexpected
    assert all("rotary" in m or "inv_freq" in m for m in missing), missing

    cache = DynamicCache(config=cfg)
    if seq_len > 0:
        kh = f(k_cache[:seq_len]).view(seq_len, NH, D).transpose(0, 1)[None]
        vh = f(v_cache[:seq_len]).view(seq_len, NH, D).transpose(0, 1)[None]
        cache.update(kh.contiguous(), vh.contiguous(), 0)
    rope = GPTNeoXRotaryEmbedding(cfg)
    hs = f(x).reshape(1, 1, H)
    pos = torch.tensor([[position]])
    with torch.no_grad():
        out = layer(hs, attention_mask=None, position_ids=pos, layer_past=cache,
                    use_cache=True, position_embeddings=rope(hs, pos))
    if isinstance(out, tuple):
        out = out[0]
    k_new = cache.layers[0].keys[:, :, -1]
    v_new = cache.layers[0].values[:, :, -1]
    return out.reshape(1, H), k_new.reshape(1, NH, D), v_new.reshape(1, NH, D)


def compare(a: torch.Tensor, b: torch.Tensor):
    """(max-abs error, relative L2 error) of a against b, both taken as fp32."""
    a = a.detach().to("cpu", torch.float32).reshape(-1)
    b = b.detach().to("cpu", torch.float32).reshape(-1)
    d = a - b
    return d.abs().max().item(), (d.norm() / b.norm().clamp_min(1e-30)).item()
