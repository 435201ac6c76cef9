"""CPU fp32 oracle for the Llama-2-7B attention-block decode step (batch 1).

TEST INFRASTRUCTURE ONLY (tests/ and nothing else import it).

Restates the torch/flashinfer reference of the reference project's own test
(tests/test_llama.py:58-110): fused add + RMSNorm (flashinfer.fused_add_rmsnorm:
residual <- input + residual in fp16, then RMSNorm with weight and eps), QKV
projection with rows [Q of all heads; K of all heads; V of all heads]
(`view(3, 32, head_dim)`, test_llama.py:64), NeoX rotate-half RoPE over the whole
head (test_llama.py:40-45), softmax(q.K^T / sqrt(D)) V over the cached rows plus the
new token (flashinfer.single_decode_with_kv_cache), output projection without bias.
The MLP is not part of the op (commented out in the reference test, :108-110).
Pinned against transformers' LlamaAttention + LlamaRMSNorm by tests/test_oracle_cpu.py.
"""
from __future__ import annotations

import math

import torch


def rotate_half(t):
    h = t.shape[-1] // 2
    return torch.cat((-t[..., h:], t[..., :h]), dim=-1)


def llama_attn_block_fp32(x, residual, weight_qkv, weight_o, k_cache, v_cache, rms_weight, eps, cos, sin,
                          heads: int = 32, head_dim: int = 128):
    """Returns (output [1,H], residual_out [1,H] (fp16-rounded values), k_new [1,NH,D], v_new [1,NH,D]) in fp32.
    k_cache / v_cache: [seq, NH*D], all rows are history; cos / sin: [D] fp32."""
    f = lambda t: t.detach().to("cpu", torch.float32)
    H = heads * head_dim
    s = (f(x).reshape(1, H) + f(residual).reshape(1, H)).to(torch.float16).to(torch.float32)
    hn = s * torch.rsqrt((s * s).mean(dim=-1, keepdim=True) + eps) * f(rms_weight).reshape(-1)
    qkv = (hn @ f(weight_qkv).t()).view(3, heads, head_dim)
    c, sn = f(cos).reshape(-1)[:head_dim], f(sin).reshape(-1)[:head_dim]
    q = qkv[0] * c + rotate_half(qkv[0]) * sn
    k_new = qkv[1] * c + rotate_half(qkv[1]) * sn
    v_new = qkv[2]
    seq = k_cache.shape[0]
    k_all = torch.cat([f(k_cache).view(seq, heads, head_dim), k_new[None]], dim=0).transpose(0, 1)
    v_all = torch.cat([f(v_cache).view(seq, heads, head_dim), v_new[None]], dim=0).transpose(0, 1)
    p = torch.softmax(torch.einsum("hd,hsd->hs", q, k_all) / math.sqrt(head_dim), dim=-1)
    attn = torch.einsum("hs,hsd->hd", p, v_all).reshape(1, H)
    return attn @ f(weight_o).t(), s, k_new[None].clone(), v_new[None].clone()


def llama_attn_block_batch_fp32(x, residual, weight_qkv, weight_o, k_pool, v_pool, indptr, indices, positions, cos_sin,
                                rms_weight, eps, heads: int = 32, head_dim: int = 128):
    """The batched, paged form of the block (llama_decoder_layer_batch_decode_sglang, include/pybind.cpp:90-106;
    page-table semantics of include/5090/llama/kernel_batch_sglang.cuh:118-123, 322-323, 343-371): sequence b owns the
    pool rows indices[indptr[b] : indptr[b+1]] (one row = one token of all heads); the LAST of them is the slot the
    new token's key / value are written to, the ones before it are its history.  cos_sin [positions, head_dim] holds
    the cos of the head_dim/2 rotation angles of a position, then their sin; positions[b] selects the row.
    Every sequence goes through llama_attn_block_fp32 (pinned against transformers) on its gathered history.
    Returns (output [B,H], residual_out [B,H], k_new [B,NH,D], v_new [B,NH,D], slots [B]) in fp32 / int64."""
    f = lambda t: t.detach().to("cpu", torch.float32)
    ip = indptr.detach().cpu().long().tolist()
    ix = indices.detach().cpu().long()
    pos = positions.detach().cpu().long().tolist()
    cs = f(cos_sin)
    half = head_dim // 2
    outs, ress, kns, vns, slots = [], [], [], [], []
    for b in range(len(ip) - 1):
        rows = ix[ip[b]:ip[b + 1] - 1]
        c, sn = cs[pos[b], :half], cs[pos[b], half:head_dim]
        o, s, kn, vn = llama_attn_block_fp32(x[b:b + 1], residual[b:b + 1], weight_qkv, weight_o, f(k_pool)[rows], f(v_pool)[rows],
                                             rms_weight, eps, torch.cat([c, c]), torch.cat([sn, sn]), heads, head_dim)
        outs.append(o), ress.append(s), kns.append(kn), vns.append(vn), slots.append(int(ix[ip[b + 1] - 1]))
    return torch.cat(outs), torch.cat(ress), torch.cat(kns), torch.cat(vns), torch.tensor(slots)


def llama_mlp_block_batch_fp32(x, residual, gate_up_weight, down_weight, rms_weight, eps):
    """llama_mlp_block_fp32 row by row: (out [B,H], residual_out [B,H])."""
    outs, ress = zip(*[llama_mlp_block_fp32(x[b:b + 1], residual[b:b + 1], gate_up_weight, down_weight, rms_weight, eps)
                       for b in range(x.shape[0])])
    return torch.cat(outs), torch.cat(ress)


def hf_llama_attn_block(x, residual, weight_qkv, weight_o, k_cache, v_cache, rms_weight, eps, cos, sin,
                        heads: int = 32, head_dim: int = 128):
    """The same block through transformers' LlamaRMSNorm + LlamaAttention (eager, fp32)."""
    from transformers import LlamaConfig
    from transformers.cache_utils import DynamicCache
    from transformers.models.llama.modeling_llama import LlamaAttention, LlamaRMSNorm
    f = lambda t: t.detach().to("cpu", torch.float32)
    H = heads * head_dim
    cfg = LlamaConfig(hidden_size=H, num_attention_heads=heads, num_key_value_heads=heads, head_dim=head_dim,
                      intermediate_size=4 * H, num_hidden_layers=1, rms_norm_eps=eps, attention_bias=False,
                      attention_dropout=0.0, vocab_size=32)
    cfg._attn_implementation = "eager"
    norm = LlamaRMSNorm(H, eps=eps).float()
    attn = LlamaAttention(cfg, layer_idx=0).float().eval()
    Wqkv = f(weight_qkv)
    with torch.no_grad():
        norm.weight.copy_(f(rms_weight).reshape(-1))
        attn.q_proj.weight.copy_(Wqkv[:H])
        attn.k_proj.weight.copy_(Wqkv[H:2 * H])
        attn.v_proj.weight.copy_(Wqkv[2 * H:])
        attn.o_proj.weight.copy_(f(weight_o))
    s = (f(x).reshape(1, H) + f(residual).reshape(1, H)).to(torch.float16).to(torch.float32)
    seq = k_cache.shape[0]
    cache = DynamicCache(config=cfg)
    cache.update(f(k_cache).view(seq, heads, head_dim).transpose(0, 1)[None].contiguous(),
                 f(v_cache).view(seq, heads, head_dim).transpose(0, 1)[None].contiguous(), 0)
    pe = (f(cos).reshape(1, 1, head_dim), f(sin).reshape(1, 1, head_dim))
    with torch.no_grad():
        out = attn(norm(s).reshape(1, 1, H), position_embeddings=pe, attention_mask=None, past_key_values=cache)[0]
    return out.reshape(1, H), s, cache.layers[0].keys[:, :, -1].reshape(1, heads, head_dim), \
        cache.layers[0].values[:, :, -1].reshape(1, heads, head_dim)


def llama_mlp_block_fp32(x, residual, gate_up_weight, down_weight, rms_weight, eps):
    """The SwiGLU MLP block with the fused-add front (same conventions as llama_attn_block_fp32):
    s = fp16(x + residual); y = RMSNorm(s) * rms_weight; out = (silu(y Wg^T) * (y Wu^T)) Wd^T.
    gate_up_weight [2F, H], gate rows first; down_weight [H, F].  Returns (out [1,H], s [1,H]) fp32.
    The reference's own test keeps this block as commented-out torch code (tests/test_llama.py:108-110);
    the arithmetic is LlamaMLP's (transformers/models/llama/modeling_llama.py)."""
    f = lambda t: t.detach().to("cpu", torch.float32)
    H = f(x).numel()
    F = down_weight.shape[-1]
    s = (f(x).reshape(1, H) + f(residual).reshape(1, H)).to(torch.float16).to(torch.float32)
    y = s * torch.rsqrt((s * s).mean(dim=-1, keepdim=True) + eps) * f(rms_weight).reshape(-1)
    gu = y @ f(gate_up_weight).t()
    mid = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    return mid @ f(down_weight).t(), s


def hf_llama_mlp_block(x, residual, gate_up_weight, down_weight, rms_weight, eps):
    """The same block through transformers' LlamaRMSNorm + LlamaMLP in fp32."""
    from transformers import LlamaConfig
    from transformers.models.llama.modeling_llama import LlamaMLP, LlamaRMSNorm
    f = lambda t: t.detach().to("cpu", torch.float32)
    H = f(x).numel()
    F = down_weight.shape[-1]
    cfg = LlamaConfig(hidden_size=H, intermediate_size=F, num_attention_heads=max(1, H // 128), num_hidden_layers=1,
                      rms_norm_eps=eps, vocab_size=32, hidden_act="silu", mlp_bias=False)
    norm = LlamaRMSNorm(H, eps=eps).float()
    mlp = LlamaMLP(cfg).float().eval()
    W = f(gate_up_weight)
    with torch.no_grad():
        norm.weight.copy_(f(rms_weight).reshape(-1))
        mlp.gate_proj.weight.copy_(W[:F])
        mlp.up_proj.weight.copy_(W[F:])
        mlp.down_proj.weight.copy_(f(down_weight))
        s = (f(x).reshape(1, H) + f(residual).reshape(1, H)).to(torch.float16).to(torch.float32)
        return mlp(norm(s)), s
