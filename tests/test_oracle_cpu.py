"""CPU checks of the oracle: against transformers' GPTNeoXLayer (the implementation
the reference's end-to-end scripts compare with) and against the committed
golden vectors."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as G  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402


@pytest.mark.parametrize("seq", [0, 5])
def test_oracle_matches_hf_layer_small(seq):
    """Same math as GPTNeoXLayer in fp32 (tanh GELU, rotary_pct 0.25, parallel residual)."""
    s = G.MINI
    w = O.make_layer_weights(s, 0, seed=5, std=0.05)
    x = O.seeded_normal((1, s.hidden), 6)
    k, v = O.make_kv_cache(s, seq, seq + 2, 7)
    cos, sin = O.rope_table(seq + 1, s.rotary)
    out, kn, vn = O.layer_decode_fp32(s, x, w, k, v, cos[seq], sin[seq], seq)
    ho, hk, hv = O.hf_layer_decode(s, x, w, k, v, seq, seq)
    for a, b in ((out, ho), (kn, hk), (vn, hv)):
        assert O.compare(a, b)[0] < 2e-5


def test_oracle_matches_hf_layer_2b8():
    s = O.PYTHIA_2B8
    s_, w, x, k, v, cos, sin = G.layer_case_inputs("2b8", 33, 1234, 7)
    out, kn, vn = O.layer_decode_fp32(s, x, w, k, v, cos, sin, 33)
    ho, hk, hv = O.hf_layer_decode(s, x, w, k, v, 33, 33)
    for a, b in ((out, ho), (kn, hk), (vn, hv)):
        assert O.compare(a, b)[0] < 2e-5


@pytest.mark.parametrize("case", [c for c in G.LAYER_CASES if c[1] == "2b8"], ids=lambda c: c[0])
def test_oracle_reproduces_golden(case):
    name, model, seq, wseed, xseed = case
    gold = np.load(os.path.join(HERE, "golden", name + ".npz"))
    s, w, x, k, v, cos, sin = G.layer_case_inputs(model, seq, wseed, xseed)
    np.testing.assert_allclose(G.checksum(x, w["qkv_weight"], w["mlp_down_weight"], k, v), gold["in_checksum"],
                               rtol=1e-9, err_msg="seeded inputs differ from the ones the golden file was made from")
    out, kn, vn = O.layer_decode_fp32(s, x, w, k, v, cos, sin, seq)
    np.testing.assert_allclose(out.numpy(), gold["out"], atol=2e-5)
    np.testing.assert_allclose(kn.numpy(), gold["k_new"], atol=2e-5)
    np.testing.assert_allclose(vn.numpy(), gold["v_new"], atol=2e-5)
    assert float(gold["hf_maxdiff"]) < 2e-5


def test_mini_rollout_golden():
    gold = np.load(os.path.join(HERE, "golden", "mini_rollout.npz"))
    prompt, tokens, gaps, logits = G.mini_rollout_oracle(round_io=False)
    assert prompt == gold["prompt"].tolist()
    assert tokens == gold["tokens"].tolist()
    assert min(gaps) > 0.01
    np.testing.assert_allclose(logits.numpy(), gold["last_logits"], atol=1e-4)


def test_rope_is_rotate_half_on_first_dims():
    """cos = 1, sin = 0 leaves q untouched; dims >= rotary always pass through
    (partial RoPE, include/5090/pythia_6b9/kernel.cuh:388-415 of the reference)."""
    t = torch.randn(4, 128)
    R = 32
    ident = O.rope_partial(t, torch.ones(R), torch.zeros(R), R)
    assert torch.equal(ident, t)
    ang = torch.rand(R)
    r = O.rope_partial(t, ang.cos(), ang.sin(), R)
    assert torch.equal(r[:, R:], t[:, R:])
    i = 3
    expect = t[:, i] * ang.cos()[i] - t[:, i + R // 2] * ang.sin()[i]
    assert torch.allclose(r[:, i], expect, atol=1e-6)
    expect2 = t[:, i + R // 2] * ang.cos()[i + R // 2] + t[:, i] * ang.sin()[i + R // 2]
    assert torch.allclose(r[:, i + R // 2], expect2, atol=1e-6)


def test_oracle_model_step_equals_layer_composition():
    s = G.MINI
    layers, head = G.mini_model()
    om = O.OracleModel(s, layers, head, 8, round_io=False)
    logits, hid = om.step(11)
    x = head["embed_in"][11].float().reshape(1, -1)
    cos, sin = O.rope_table(8, s.rotary)
    for w in layers:
        x, _, _ = O.layer_decode_fp32(s, x, w, torch.zeros(8, s.heads * s.head_dim), torch.zeros(8, s.heads * s.head_dim),
                                      cos[0], sin[0], 0)
    assert torch.allclose(hid, x, atol=1e-6)
    assert torch.allclose(logits, O.final_logits_fp32(x, head).reshape(-1), atol=1e-6)


def test_llama_oracle_matches_hf_attention():
    """The Llama attention-block restatement against transformers' LlamaRMSNorm + LlamaAttention."""
    from oracle import llama_oracle as L
    NH, D, seq = 4, 32, 9
    H = NH * D
    x, r = O.seeded_normal((1, H), 1), O.seeded_normal((1, H), 2)
    wq, wo = O.seeded_normal((3 * H, H), 3, std=0.1), O.seeded_normal((H, H), 4, std=0.1)
    g = O.seeded_normal((H,), 5, mean=1.0, std=0.1)
    k, v = O.seeded_normal((seq, H), 6), O.seeded_normal((seq, H), 7)
    ang = torch.rand(D // 2, generator=torch.Generator().manual_seed(8)) * 6.28
    cos, sin = torch.cat([ang.cos(), ang.cos()]), torch.cat([ang.sin(), ang.sin()])
    a = L.llama_attn_block_fp32(x, r, wq, wo, k, v, g, 1e-6, cos, sin, NH, D)
    b = L.hf_llama_attn_block(x, r, wq, wo, k, v, g, 1e-6, cos, sin, NH, D)
    for p, q in zip(a, b):
        assert O.compare(p, q)[0] < 1e-5


def test_llama_mlp_oracle_matches_hf_mlp():
    """Pins the SwiGLU MLP restatement against transformers' LlamaRMSNorm + LlamaMLP (fp32)."""
    from oracle import llama_oracle as L
    g = torch.Generator().manual_seed(11)
    H, F = 512, 1408
    rw = lambda *shape: (torch.randn(*shape, generator=g) * 0.1).half()
    x, r, wgu, wd, gm = rw(1, H), rw(1, H), rw(2 * F, H), rw(H, F), rw(1, H)
    a = L.llama_mlp_block_fp32(x, r, wgu, wd, gm, 1e-6)
    b = L.hf_llama_mlp_block(x, r, wgu, wd, gm, 1e-6)
    assert torch.equal(a[1], b[1])
    assert torch.allclose(a[0], b[0], atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("case", G.LLAMA_ATTN_CASES + G.LLAMA_MLP_CASES, ids=lambda c: c[0])
def test_llama_oracle_reproduces_golden(case):
    """The Llama restatements against the committed fixtures (made by tests/golden/make_golden.py, where
    they were also cross-checked against transformers' LlamaAttention / LlamaMLP)."""
    from oracle import llama_oracle as L
    name, size, seed = case
    gold = np.load(os.path.join(HERE, "golden", name + ".npz"))
    assert float(gold["hf_maxdiff"]) < 2e-5
    if name.startswith("llama_attn"):
        t = G.llama_attn_inputs(size, seed)
        np.testing.assert_allclose(G.checksum(t["x"], t["wqkv"], t["wo"], t["k"], t["v"]), gold["in_checksum"], rtol=1e-9)
        out, res, kn, vn = L.llama_attn_block_fp32(t["x"], t["res"], t["wqkv"], t["wo"], t["k"], t["v"], t["g"],
                                                   G.LLAMA_EPS, t["cos"], t["sin"])
        np.testing.assert_allclose(kn.numpy(), gold["k_new"], atol=1e-5, rtol=1e-5)
        np.testing.assert_allclose(vn.numpy(), gold["v_new"], atol=1e-5, rtol=1e-5)
    else:
        t = G.llama_mlp_inputs(size, seed)
        np.testing.assert_allclose(G.checksum(t["x"], t["wgu"], t["wd"]), gold["in_checksum"], rtol=1e-9)
        out, res = L.llama_mlp_block_fp32(t["x"], t["res"], t["wgu"], t["wd"], t["g"], G.LLAMA_EPS)
    np.testing.assert_array_equal(res.numpy(), gold["residual"])
    np.testing.assert_allclose(out.numpy(), gold["out"], atol=1e-5, rtol=1e-5)


def test_llama_batch_oracle_gathers_through_the_page_table():
    """The batched oracle is the pinned single-sequence oracle applied to every sequence's gathered history: a
    shuffled page table must give the same result as contiguous caches, and the slot is the sequence's last entry."""
    from oracle import llama_oracle as LO
    torch.manual_seed(0)
    heads, hd = 4, 128
    Hs = heads * hd
    lengths = [5, 0, 9]
    wqkv, wo = torch.randn(3 * Hs, Hs) * 0.05, torch.randn(Hs, Hs) * 0.05
    g1 = 1 + 0.02 * torch.randn(Hs)
    n_rows = sum(lengths) + len(lengths) + 3
    kpool, vpool = torch.randn(n_rows, Hs).half(), torch.randn(n_rows, Hs).half()
    perm = torch.randperm(n_rows)
    indptr, idx, at = [0], [], 0
    for s_ in lengths:
        idx.append(perm[at:at + s_ + 1]); at += s_ + 1; indptr.append(indptr[-1] + s_ + 1)
    indices = torch.cat(idx)
    x, res = torch.randn(3, Hs).half(), torch.randn(3, Hs).half()
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    ang = torch.outer(torch.arange(16).float(), inv)
    cs = torch.cat([ang.cos(), ang.sin()], dim=1)
    pos = torch.tensor(lengths)
    o, s, kn, vn, slots = LO.llama_attn_block_batch_fp32(x, res, wqkv, wo, kpool, vpool, torch.tensor(indptr), indices, pos, cs,
                                                         g1, 1e-5, heads, hd)
    assert slots.tolist() == [int(indices[indptr[b + 1] - 1]) for b in range(3)]
    for b, s_ in enumerate(lengths):
        rows = indices[indptr[b]:indptr[b] + s_]
        c, sn = torch.cat([cs[s_, :64], cs[s_, :64]]), torch.cat([cs[s_, 64:], cs[s_, 64:]])
        ob, sb, kb, vb = LO.llama_attn_block_fp32(x[b:b + 1], res[b:b + 1], wqkv, wo, kpool[rows], vpool[rows], g1, 1e-5, c, sn, heads, hd)
        assert torch.equal(o[b:b + 1], ob) and torch.equal(kn[b:b + 1], kb) and torch.equal(s[b:b + 1], sb)
