"""Whole-model greedy decode (embedding -> layers -> final LayerNorm -> LM head -> argmax
as one launch per token) against the fp32 oracle and against the per-layer op."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, HERE)
import make_golden as G  # noqa: E402
from _util import MAX_ABS, REL_L2, assert_close, layer_args  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def dims_of(shape):
    import clusterfusion as cf
    d = cf.CfDims()
    d.hidden, d.heads, d.head_dim, d.rotary, d.ffn, d.vocab = (shape.hidden, shape.heads, shape.head_dim, shape.rotary,
                                                               shape.ffn, shape.vocab)
    return d


def build_decoder(shape, layers, head, max_seq, dev, use_graph):
    import clusterfusion as cf
    KVW = shape.heads * shape.head_dim
    caches = [(torch.zeros(max_seq, KVW, dtype=torch.float16, device=dev),
               torch.zeros(max_seq, KVW, dtype=torch.float16, device=dev)) for _ in layers]
    ld = [{n: t.to(dev) for n, t in w.items()} for w in layers]
    hd = {n: t.to(dev) for n, t in head.items()}
    return cf.PythiaDecoder(dims_of(shape), ld, hd, caches, max_seq, use_graph=use_graph), ld, hd, caches


@pytest.mark.parametrize("use_graph", [False, True])
def test_mini_rollout_tokens_match_golden(cuda_device, use_graph):
    """Prompt + 24 greedy steps of a 3-layer model: token ids identical to the committed
    fp32 oracle rollout, final logits within tolerance."""
    import clusterfusion as cf
    gold = np.load(os.path.join(HERE, "golden", "mini_rollout.npz"))
    layers, head = G.mini_model()
    cfg = G.MINI_ROLLOUT
    max_seq = cfg["prompt_len"] + cfg["steps"] + 2
    dec, *_ = build_decoder(G.MINI, layers, head, max_seq, cuda_device, use_graph)
    prompt = gold["prompt"].tolist()
    dec.reset(0, prompt[0])
    for i, t in enumerate(prompt):          # prompt ingestion token by token (teacher forced)
        dec.token.fill_(t)
        dec.step()
    toks = []
    tok = int(dec.token.item())
    for _ in range(cfg["steps"]):
        toks.append(tok)
        dec.step()
        tok = int(dec.token.item())
    assert toks == gold["tokens"].tolist()
    assert int(dec.seq_len.item()) == cfg["prompt_len"] + cfg["steps"]
    mx, rl = O.compare(dec.logits, torch.from_numpy(gold["last_logits"]))
    assert mx <= MAX_ABS and rl <= 5 * REL_L2, (mx, rl)
    assert cf.device_status() == 0
    dec.close()


def test_decoder_equals_per_layer_op(cuda_device):
    """One launch for the whole token == the per-layer op called layer by layer + torch tail,
    bit for bit on the hidden state (same kernels, same reduction order)."""
    import clusterfusion as cf
    s = O.Shape("2b8-4l", 2560, 32, 80, 20, 10240, 50304, layers=4)
    layers = [O.make_layer_weights(s, l, seed=77, device=cuda_device) for l in range(s.layers)]
    head = O.make_head_weights(s, seed=77, device=cuda_device)
    ctx, max_seq = 300, 310
    dec, ld, hd, caches = build_decoder(s, layers, head, max_seq, cuda_device, use_graph=False)
    for l, (k, v) in enumerate(caches):
        kk, vv = O.make_kv_cache(s, ctx, max_seq, 500 + l, device=cuda_device)
        k.copy_(kk), v.copy_(vv)
    ref_caches = [(k.clone(), v.clone()) for k, v in caches]
    cos_t, sin_t = O.rope_table(max_seq, s.rotary, device=cuda_device)
    tok = 4242
    dec.reset(ctx, tok)
    for step in range(3):
        pos = ctx + step
        dec.step()
        h = hd["embed_in"][tok].reshape(1, -1).contiguous()
        for l, w in enumerate(ld):
            h, _, _ = cf.pythia_2b8_decoder_layer(*layer_args(h, w, ref_caches[l][0], ref_caches[l][1],
                                                              cos_t[pos].contiguous(), sin_t[pos].contiguous(), pos))
        assert torch.equal(dec.hidden, h)
        ref_logits = O.final_logits_fp32(h, hd).reshape(-1)
        mx, rl = O.compare(dec.logits, ref_logits)
        assert mx <= 2e-3 and rl <= 1e-4, (mx, rl)
        tok = int(dec.token.item())
        assert tok == int(dec.logits.argmax().item())
    for (k, v), (kr, vr) in zip(caches, ref_caches):
        assert torch.equal(k, kr) and torch.equal(v, vr)
    assert cf.device_status() == 0
    dec.close()


def _full_model_rollout(shape, prompt_len, steps, seed, dev):
    """Oracle prefill + greedy rollout in fp32 on the CPU vs the decoder on the GPU."""
    import clusterfusion as cf
    layers = [O.make_layer_weights(shape, l, seed=seed, device=dev) for l in range(shape.layers)]
    head = O.make_head_weights(shape, seed=seed, device=dev)
    max_seq = prompt_len + steps + 2
    om = O.OracleModel(shape, [{n: t.cpu() for n, t in w.items()} for w in layers],
                       {n: t.cpu() for n, t in head.items()}, max_seq, round_io=False)
    g = torch.Generator().manual_seed(seed)
    prompt = torch.randint(0, shape.vocab, (prompt_len,), generator=g).tolist()
    logits = None
    for t in prompt:
        logits, _ = om.step(t)
    dec, ld, hd, caches = build_decoder(shape, layers, head, max_seq, dev, use_graph=True)
    for l, (k, v) in enumerate(caches):      # prefill by the oracle, cast to fp16 on both sides
        k[:prompt_len] = om.k[l][:prompt_len].half().to(dev)
        v[:prompt_len] = om.v[l][:prompt_len].half().to(dev)
        om.k[l][:prompt_len] = om.k[l][:prompt_len].half().float()
        om.v[l][:prompt_len] = om.v[l][:prompt_len].half().float()
    tok = int(logits.argmax())
    dec.reset(prompt_len, tok)
    got, want, gaps = [], [], []
    otok = tok
    for _ in range(steps):
        dec.step()
        got.append(int(dec.token.item()))
        logits, _ = om.step(otok)
        top2 = torch.topk(logits, 2).values
        gaps.append((top2[0] - top2[1]).item())
        otok = int(logits.argmax())
        want.append(otok)
    status = cf.device_status()
    mx, rl = O.compare(dec.logits, logits)
    dec.close()
    return got, want, gaps, (mx, rl), status


def test_pythia_2b8_greedy_64_steps_identical(cuda_device):
    """The full-model parity case (full Pythia-2.8B, seeded random init, prompt of 128 random
    ids): 64 greedy tokens identical to the fp32 oracle's."""
    got, want, gaps, (mx, rl), status = _full_model_rollout(O.PYTHIA_2B8, 128, 64, 31337, cuda_device)
    first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
    assert status == 0
    assert got == want, f"first mismatch at step {first_diff}; min top-2 gap of the oracle {min(gaps):.4g}, " \
                        f"gap at mismatch {gaps[first_diff]:.4g}"
    assert mx <= MAX_ABS and rl <= 5 * REL_L2, (mx, rl)


def test_pythia_6b9_shapes_greedy_64_steps_identical(cuda_device):
    """The configuration the headline number is timed on, as a parity case: Pythia-6.9B layer shapes
    (hidden 4096, 32 heads x 128, ffn 16384, vocabulary 50432), 8 layers, every cache filled to 4096
    rows of N(0, 1) fp16 history (33 attention chunks per head), whole-token launches replayed from a
    CUDA graph: 64 greedy tokens identical to the fp32 oracle's on the same seeded tensors."""
    import clusterfusion as cf
    dev = cuda_device
    shape = O.Shape("6b9-8l", 4096, 32, 128, 32, 16384, 50432, layers=8)
    seed, ctx, steps = 2024, 4096, 64
    layers = [O.make_layer_weights(shape, l, seed=seed, device=dev) for l in range(shape.layers)]
    head = O.make_head_weights(shape, seed=seed, device=dev)
    max_seq = ctx + steps + 2
    om = O.OracleModel(shape, [{n: t.cpu() for n, t in w.items()} for w in layers],
                       {n: t.cpu() for n, t in head.items()}, max_seq, round_io=False)
    dec, ld, hd, caches = build_decoder(shape, layers, head, max_seq, dev, use_graph=True)
    for l, (k, v) in enumerate(caches):
        kk, vv = O.make_kv_cache(shape, ctx, max_seq, 900 + l, device=dev)
        k.copy_(kk), v.copy_(vv)
        om.load_cache(l, kk, vv, ctx)
    om.seq_len = ctx
    tok = otok = 4242
    dec.reset(ctx, tok)
    got, want, gaps = [], [], []
    logits = None
    for _ in range(steps):
        dec.step()
        got.append(int(dec.token.item()))
        logits, _ = om.step(otok)
        top2 = torch.topk(logits, 2).values
        gaps.append((top2[0] - top2[1]).item())
        otok = int(logits.argmax())
        want.append(otok)
    status = cf.device_status()
    mx, rl = O.compare(dec.logits, logits)
    dec.close()
    first_diff = next((i for i, (a, b) in enumerate(zip(got, want)) if a != b), None)
    assert status == 0
    assert got == want, f"first mismatch at step {first_diff}; min top-2 gap of the oracle {min(gaps):.4g}, " \
                        f"gap at mismatch {gaps[first_diff]:.4g}"
    assert mx <= MAX_ABS and rl <= 5 * REL_L2, (mx, rl)


def test_few_heads_long_context_merge_paths(cuda_device, monkeypatch):
    """A model with 4 heads (the shape of one rank's shard at 8-way tensor parallelism) and 1 200 cached rows:
    every head's attention is split into ~10 partial records on as many CTAs, the table of partials per head is
    long (39 slots), so the merge cuts each vector's records into segments summed by different helper threads.
    32 greedy tokens identical to the fp32 oracle's; and the same tokens, logits within 1e-3, when the segment
    count is capped at 1 (CFB200_MERGE_SEG=1: every record of a vector summed by one thread in slot order)."""
    import clusterfusion as cf
    dev = cuda_device
    shape = O.Shape("few-heads", 512, 4, 128, 32, 1024, 1024, layers=3)
    seed, ctx, steps = 77, 1200, 32
    layers = [O.make_layer_weights(shape, l, seed=seed, device=dev) for l in range(shape.layers)]
    head = O.make_head_weights(shape, seed=seed, device=dev)
    max_seq = ctx + steps + 2
    om = O.OracleModel(shape, [{n: t.cpu() for n, t in w.items()} for w in layers],
                       {n: t.cpu() for n, t in head.items()}, max_seq, round_io=False)
    kv = [O.make_kv_cache(shape, ctx, max_seq, 500 + l, device=dev) for l in range(shape.layers)]
    for l, (kk, vv) in enumerate(kv):
        om.load_cache(l, kk, vv, ctx)
    om.seq_len = ctx
    want, otok = [], 99
    logits = None
    for _ in range(steps):
        logits, _ = om.step(otok)
        otok = int(logits.argmax())
        want.append(otok)

    def rollout(cap):
        monkeypatch.setenv("CFB200_MERGE_SEG", str(cap))
        dec, ld, hd, caches = build_decoder(shape, layers, head, max_seq, dev, use_graph=False)
        for (k, v), (kk, vv) in zip(caches, kv):
            k.copy_(kk), v.copy_(vv)
        dec.reset(ctx, 99)
        got = []
        for _ in range(steps):
            dec.step()
            got.append(int(dec.token.item()))
        out = dec.logits.float().cpu().clone()
        dec.close()
        return got, out

    try:
        got_seg, log_seg = rollout(0)     # automatic: five segments per vector
        got_one, log_one = rollout(1)     # one segment
    finally:
        monkeypatch.setenv("CFB200_MERGE_SEG", "0")
    assert cf.device_status() == 0
    assert got_seg == want, (got_seg, want)
    assert got_one == want
    mx, rl = O.compare(log_seg, logits)
    assert mx <= MAX_ABS and rl <= 5 * REL_L2, (mx, rl)
    assert (log_seg - log_one).abs().max().item() <= 1e-3
