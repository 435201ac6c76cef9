"""Llama-2-7B attention block (llama_decoder_layer_sglang) against the fp32 CPU oracle,
mirroring the reference's tests/test_llama.py (randn * 0.1 tensors, random RoPE angles,
cos/sin = cat(c, c), eps 1e-6; its pass rule is average MAE < 0.01)."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _util import REL_L2, assert_close  # noqa: E402
from oracle import llama_oracle as L  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

sys.path.insert(0, os.path.join(HERE, "golden"))
import make_golden as G  # noqa: E402

pytestmark = pytest.mark.gpu
H, NH, D = 4096, 32, 128


def make(seq, dev, seed=42):
    g = torch.Generator(device=dev).manual_seed(seed)
    rw = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.1).half()
    t = dict(x=rw(1, H), res=rw(1, H), wqkv=rw(3 * H, H), wo=rw(H, H), k=rw(seq, H), v=rw(seq, H), g=rw(1, H))
    ang = torch.rand(D // 2, generator=g, device=dev) * (2 * torch.pi)
    t["cos"] = torch.cat([ang.cos(), ang.cos()]).contiguous()
    t["sin"] = torch.cat([ang.sin(), ang.sin()]).contiguous()
    return t


@pytest.mark.parametrize("seq", [1, 63, 64, 65, 1000, 2048, 4096])
def test_llama_attention_block_vs_oracle(cuda_device, seq):
    import clusterfusion as cf
    t = make(seq, cuda_device)
    res_in = t["res"].clone()
    k0, v0 = t["k"].clone(), t["v"].clone()
    out, res, kn, vn = cf.llama_decoder_layer_sglang(t["x"], t["res"], t["wqkv"], t["wo"], t["k"], t["v"], t["g"], 1e-6,
                                                     t["cos"], t["sin"])
    assert cf.device_status() == 0
    assert res.data_ptr() == t["res"].data_ptr()          # updated in place and returned
    ro, rr, rk, rv = L.llama_attn_block_fp32(t["x"], res_in, t["wqkv"], t["wo"], k0, v0, t["g"], 1e-6, t["cos"], t["sin"])
    assert torch.equal(res.float().cpu(), rr)              # fp16 sum, exact
    mae = (out.float().cpu() - ro).abs().mean().item()
    assert mae < 0.01                                       # the reference's own bar
    assert O.compare(out, ro)[1] <= REL_L2
    assert_close(kn, rk, "k_new")
    assert_close(vn, rv, "v_new")
    assert torch.equal(t["k"], k0) and torch.equal(t["v"], v0)   # caches are read-only for this op


def test_llama_block_over_growing_caches_needs_no_upload(cuda_device):
    """A decode loop hands this entry point caches of exactly seq_len rows, one row longer every token
    (include/5090/llama/llama_kernel_dispatch.cu:35 takes SEQ_LEN from k_cache.size(0)).  The key / value
    tensor maps travel in the kernel parameters, so after the first call with a set of weights nothing is
    uploaded any more: every later length can be CAPTURED into a CUDA graph (an upload would be refused there)
    and the replay matches the eager call and the oracle."""
    import clusterfusion as cf
    t = make(300, cuda_device, seed=9)
    cf.llama_decoder_layer_sglang(t["x"], t["res"].clone(), t["wqkv"], t["wo"], t["k"][:200], t["v"][:200], t["g"], 1e-6,
                                  t["cos"], t["sin"])             # first call with these weights: descriptor upload
    torch.cuda.synchronize()
    for seq in (201, 202, 257, 300):
        k, v = t["k"][:seq], t["v"][:seq]
        eager = cf.llama_decoder_layer_sglang(t["x"], t["res"].clone(), t["wqkv"], t["wo"], k, v, t["g"], 1e-6, t["cos"], t["sin"])
        eager = [e.clone() for e in eager]
        res = t["res"].clone()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = cf.llama_decoder_layer_sglang(t["x"], res, t["wqkv"], t["wo"], k, v, t["g"], 1e-6, t["cos"], t["sin"])
        res.copy_(t["res"])
        g.replay()
        torch.cuda.synchronize()
        for a, b in zip(out, eager):
            assert torch.equal(a, b)
        ro, _, _, _ = L.llama_attn_block_fp32(t["x"], t["res"], t["wqkv"], t["wo"], k, v, t["g"], 1e-6, t["cos"], t["sin"])
        assert O.compare(out[0], ro)[1] <= REL_L2
    assert cf.device_status() == 0


def test_llama_deterministic_and_checked(cuda_device):
    import clusterfusion as cf
    t = make(777, cuda_device, seed=1)
    first = None
    for _ in range(10):
        out, _, kn, vn = cf.llama_decoder_layer_sglang(t["x"], t["res"].clone(), t["wqkv"], t["wo"], t["k"], t["v"],
                                                       t["g"], 1e-6, t["cos"], t["sin"])
        if first is None:
            first = out.clone()
        assert torch.equal(out, first)
    with pytest.raises(RuntimeError):
        cf.llama_decoder_layer_sglang(t["x"].float(), t["res"], t["wqkv"], t["wo"], t["k"], t["v"], t["g"], 1e-6,
                                      t["cos"], t["sin"])
    with pytest.raises(RuntimeError):
        cf.llama_decoder_layer_sglang(t["x"], t["res"], t["wqkv"], t["wo"], t["k"][:0], t["v"][:0], t["g"], 1e-6,
                                      t["cos"], t["sin"])


def make_mlp(ffn, dev, seed=7):
    g = torch.Generator(device=dev).manual_seed(seed)
    rw = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.1).half()
    # weights at the scale of a trained model keep |out| ~ 1, where the absolute tolerance means something
    rs = lambda *shape: (torch.randn(*shape, generator=g, device=dev) * 0.02).half()
    return dict(x=rw(1, H), res=rw(1, H), wgu=rs(2 * ffn, H), wd=rs(H, ffn), g=(1 + 0.1 * torch.randn(1, H, generator=g, device=dev)).half())


@pytest.mark.parametrize("ffn", [11008, 8192, 2048, 5504])
def test_llama_mlp_block_vs_oracle(cuda_device, ffn):
    import clusterfusion as cf
    t = make_mlp(ffn, cuda_device)
    res_in = t["res"].clone()
    out, res = cf.llama_mlp_sglang(t["x"], t["res"], t["wgu"], t["wd"], t["g"], 1e-5)
    assert cf.device_status() == 0
    assert res.data_ptr() == t["res"].data_ptr()
    ro, rr = L.llama_mlp_block_fp32(t["x"], res_in, t["wgu"], t["wd"], t["g"], 1e-5)
    assert torch.equal(res.float().cpu(), rr)
    assert_close(out, ro, "mlp output")
    again, _ = cf.llama_mlp_sglang(t["x"], res_in.clone(), t["wgu"], t["wd"], t["g"], 1e-5)
    assert torch.equal(out, again)                         # deterministic


def test_llama_layer_stack_two_layers_vs_oracle(cuda_device):
    """Attention block then MLP block, twice, with the (hidden, residual) hand-over serving stacks use."""
    import clusterfusion as cf
    seq, ffn = 300, 11008
    layers = [(make(seq, cuda_device, seed=20 + i), make_mlp(ffn, cuda_device, seed=30 + i)) for i in range(2)]
    for a, _ in layers:  # trained-model scale for the attention weights too
        a["wqkv"] = (a["wqkv"].float() * 0.2).half()
        a["wo"] = (a["wo"].float() * 0.2).half()
    x = layers[0][0]["x"].clone()
    res = layers[0][0]["res"].clone()
    xo, ro = x.clone(), res.clone()
    for a, m in layers:
        x, res, _, _ = cf.llama_decoder_layer_sglang(x, res, a["wqkv"], a["wo"], a["k"], a["v"], a["g"], 1e-5, a["cos"], a["sin"])
        x, res = cf.llama_mlp_sglang(x, res, m["wgu"], m["wd"], m["g"], 1e-5)
        xo, ro, _, _ = L.llama_attn_block_fp32(xo, ro, a["wqkv"], a["wo"], a["k"], a["v"], a["g"], 1e-5, a["cos"], a["sin"])
        xo = xo.half()
        xo, ro = L.llama_mlp_block_fp32(xo, ro, m["wgu"], m["wd"], m["g"], 1e-5)
        xo = xo.half()
    assert cf.device_status() == 0
    assert_close(x, xo.float(), "stack output")
    assert_close(res, ro, "stack residual")


@pytest.mark.parametrize("one_launch", [False, True], ids=["per-block", "one-launch"])
def test_llama_layer_stack_class_matches_block_calls(cuda_device, one_launch):
    """LlamaLayerStack (ping-pong buffers, no copies) gives bit-identical results to chaining the two block calls --
    launched block by block, and with all blocks of the step recorded and run as ONE persistent launch
    (cf_batch_begin / cf_batch_end: grid barriers between the blocks), twice (the second batch is identical and
    needs no upload) and captured into a CUDA graph."""
    import clusterfusion as cf
    seq, ffn = 129, 11008
    blocks = [(make(seq, cuda_device, seed=40 + i), make_mlp(ffn, cuda_device, seed=50 + i)) for i in range(3)]
    layers = [dict(weight_qkv=a["wqkv"], weight_o=a["wo"], rms_input_weight=a["g"], k_cache=a["k"], v_cache=a["v"],
                   gate_up_weight=m["wgu"], down_weight=m["wd"], rms_post_weight=m["g"]) for a, m in blocks]
    a0 = blocks[0][0]
    stack = cf.LlamaLayerStack(layers, eps=1e-5, one_launch=one_launch)
    xs, rs = stack.step(a0["x"], a0["res"], a0["cos"], a0["sin"])
    if one_launch:
        first = (xs.clone(), rs.clone())
        xs, rs = stack.step(a0["x"], a0["res"], a0["cos"], a0["sin"])
        assert torch.equal(xs, first[0]) and torch.equal(rs, first[1])
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            stack.step(a0["x"], a0["res"], a0["cos"], a0["sin"])
        xs.zero_(), rs.zero_()
        g.replay()
        torch.cuda.synchronize()
        assert torch.equal(xs, first[0]) and torch.equal(rs, first[1])
    x, res = a0["x"].clone(), a0["res"].clone()
    for i, (a, m) in enumerate(blocks):
        x, res, kn, vn = cf.llama_decoder_layer_sglang(x, res, a["wqkv"], a["wo"], a["k"], a["v"], a["g"], 1e-5, a0["cos"], a0["sin"])
        assert torch.equal(kn[0], stack.k_new[i]) and torch.equal(vn[0], stack.v_new[i])
        x, res = cf.llama_mlp_sglang(x, res, m["wgu"], m["wd"], m["g"], 1e-5)
    assert torch.equal(x, xs) and torch.equal(res, rs)
    assert cf.device_status() == 0


@pytest.mark.parametrize("case", G.LLAMA_ATTN_CASES + G.LLAMA_MLP_CASES, ids=lambda c: c[0])
def test_llama_blocks_vs_golden_fixture(cuda_device, case):
    """The kernels against the committed fixtures: inputs regenerated from the seed on the CPU, moved to the GPU."""
    import numpy as np
    import clusterfusion as cf
    name, size, seed = case
    gold = np.load(os.path.join(HERE, "golden", name + ".npz"))
    if name.startswith("llama_attn"):
        t = {k: v.to(cuda_device) for k, v in G.llama_attn_inputs(size, seed).items()}
        out, res, kn, vn = cf.llama_decoder_layer_sglang(t["x"], t["res"], t["wqkv"], t["wo"], t["k"], t["v"], t["g"],
                                                         G.LLAMA_EPS, t["cos"], t["sin"])
        assert_close(kn, torch.from_numpy(gold["k_new"]), "k_new")
        assert_close(vn, torch.from_numpy(gold["v_new"]), "v_new")
    else:
        t = {k: v.to(cuda_device) for k, v in G.llama_mlp_inputs(size, seed).items()}
        out, res = cf.llama_mlp_sglang(t["x"], t["res"], t["wgu"], t["wd"], t["g"], G.LLAMA_EPS)
    assert cf.device_status() == 0
    assert torch.equal(res.float().cpu(), torch.from_numpy(gold["residual"]))
    assert_close(out, torch.from_numpy(gold["out"]), "output")
