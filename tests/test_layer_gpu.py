"""Parity of the fused decoder-layer op with the fp32 CPU oracle, on the GPU,
through the C ABI.  Mirrors the reference's tests/test_pythia.py and
tests/test_pythia_6b9.py (one layer, synthetic weights, compare with a torch
reference) with the bar of this build: max-abs <= 2e-2 and relative L2 <= 1e-3 on
the output hidden state AND on k_new / v_new (which the reference never checks)."""
import os
import sys

import numpy as np
import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, HERE)
import make_golden as G  # noqa: E402
from _util import MAX_ABS, REL_L2, assert_close, layer_args, make_case  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def fn_for(model, split=False):
    import clusterfusion as cf
    return {("2b8", False): cf.pythia_2b8_decoder_layer, ("2b8", True): cf.pythia_2b8_decoder_layer_split,
            ("6b9", False): cf.pythia_6b9_decoder_layer, ("6b9", True): cf.pythia_6b9_decoder_layer_split}[(model, split)]


def run_and_check(model, seq, rows=None, split=False, **kw):
    import clusterfusion as cf
    s, w, x, k, v, cos, sin = make_case(model, seq, rows, **kw)
    k0, v0 = k.clone(), v.clone()
    out, kn, vn = fn_for(model, split)(*layer_args(x, w, k, v, cos, sin, seq))
    assert cf.device_status() == 0
    assert out.shape == (1, s.hidden) and kn.shape == (1, s.heads, s.head_dim) and vn.shape == kn.shape
    assert out.dtype == torch.float16
    ro, rk, rv = O.layer_decode_fp32(s, x, w, k0, v0, cos, sin, seq)
    assert_close(out, ro, f"{model} seq {seq} output")
    assert_close(kn, rk, f"{model} seq {seq} k_new")
    assert_close(vn, rv, f"{model} seq {seq} v_new")
    # side effect of the op: row seq_len of both caches, nothing else
    assert torch.equal(k[seq].view(-1), kn.view(-1)) and torch.equal(v[seq].view(-1), vn.view(-1))
    keep = torch.ones(k.shape[0], dtype=torch.bool, device=k.device)
    keep[seq] = False
    assert torch.equal(k[keep], k0[keep]) and torch.equal(v[keep], v0[keep])
    return out, kn, vn


# empty cache, tile edges of the 128-row attention chunks (and of the earlier 64-row ones), the reference test's 129, a full config-1 cache
@pytest.mark.parametrize("seq", [0, 1, 2, 31, 32, 33, 63, 64, 65, 127, 128, 129, 200, 255, 256, 257, 1024, 4095])
def test_layer_2b8_vs_oracle(cuda_device, seq):
    run_and_check("2b8", seq)


@pytest.mark.parametrize("seq", [0, 1, 63, 64, 65, 129, 1024, 4096])
def test_layer_6b9_vs_oracle(cuda_device, seq):
    run_and_check("6b9", seq)


def test_layer_6b9_long_context(cuda_device):
    run_and_check("6b9", 8192, rows=8192 + 256)


def test_last_row_of_cache_is_usable(cuda_device):
    run_and_check("2b8", 99, rows=100)


@pytest.mark.parametrize("case", G.LAYER_CASES, ids=lambda c: c[0])
def test_layer_vs_golden_fixture(cuda_device, case):
    """Against the committed fp32 oracle outputs (inputs regenerated from their seeds on the CPU)."""
    name, model, seq, wseed, xseed = case
    gold = np.load(os.path.join(HERE, "golden", name + ".npz"))
    s, w, x, k, v, cos, sin = G.layer_case_inputs(model, seq, wseed, xseed)
    np.testing.assert_allclose(G.checksum(x, w["qkv_weight"], w["mlp_down_weight"], k, v), gold["in_checksum"], rtol=1e-9)
    dev = cuda_device
    wd = {n: t.to(dev) for n, t in w.items()}
    out, kn, vn = fn_for(model)(*layer_args(x.to(dev), wd, k.to(dev), v.to(dev), cos.to(dev), sin.to(dev), seq))
    assert_close(out, torch.from_numpy(gold["out"]), name + " output")
    assert_close(kn, torch.from_numpy(gold["k_new"]), name + " k_new")
    assert_close(vn, torch.from_numpy(gold["v_new"]), name + " v_new")


def test_reference_style_unit_test(cuda_device):
    """The reference's own unit test: seqlen 129, everything randn * 0.1, random RoPE angles,
    pass rule average MAE < 0.01 (tests/test_pythia_6b9.py:183-185,42-50,313-319) -- here
    against the fp32 oracle and with the tighter bar as well."""
    import clusterfusion as cf
    s = O.PYTHIA_6B9
    g = torch.Generator(device="cuda").manual_seed(42)
    rw = lambda *shape: (torch.randn(*shape, generator=g, device="cuda") * 0.1).half()
    H, F, seq = s.hidden, s.ffn, 129
    w = dict(qkv_weight=rw(3 * H, H), qkv_bias=rw(3 * H), o_weight=rw(H, H), o_bias=rw(H), ln_weight=rw(H), ln_bias=rw(H),
             post_ln_weight=rw(H), post_ln_bias=rw(H), mlp_up_weight=rw(F, H), mlp_up_bias=rw(F),
             mlp_down_weight=rw(H, F), mlp_down_bias=rw(H))
    x = rw(1, H)
    k, v = rw(seq + 1, H), rw(seq + 1, H)
    ang = torch.rand(s.rotary, generator=g, device="cuda") * (2 * torch.pi)
    cos, sin = ang.cos().contiguous(), ang.sin().contiguous()
    k0, v0 = k.clone(), v.clone()
    out, kn, vn = cf.pythia_6b9_decoder_layer(*layer_args(x, w, k, v, cos, sin, seq))
    ro, rk, rv = O.layer_decode_fp32(s, x, w, k0, v0, cos, sin, seq)
    mae = (out.float().cpu() - ro).abs().mean().item()
    assert mae < 0.01
    # output magnitude here is ~10, so the relative bar is the meaningful one
    assert O.compare(out, ro)[1] <= REL_L2
    assert_close(kn, rk, "k_new")
    assert_close(vn, rv, "v_new")


def test_cos_sin_padded_to_head_dim(cuda_device):
    """The 2.8B caller of the reference passes cos/sin as [1, head_dim] padded with cos=1, sin=0
    (tests/test_pythia.py:34-42); only the first `rotary` entries may be read."""
    import clusterfusion as cf
    s, w, x, k, v, cos, sin = make_case("2b8", 40)
    pad = s.head_dim - s.rotary
    cos_p = torch.cat([cos, torch.full((pad,), 123.0, device=cos.device)]).reshape(1, -1).contiguous()
    sin_p = torch.cat([sin, torch.full((pad,), -77.0, device=cos.device)]).reshape(1, -1).contiguous()
    k2, v2 = k.clone(), v.clone()
    a = cf.pythia_2b8_decoder_layer(*layer_args(x, w, k, v, cos, sin, 40))
    b = cf.pythia_2b8_decoder_layer(*layer_args(x, w, k2, v2, cos_p, sin_p, 40))
    for t, u in zip(a, b):
        assert torch.equal(t, u)


def test_ln_params_as_row_vectors(cuda_device):
    """ln weights may come as [1, H] (tests/test_pythia_6b9.py:197-204 builds them that way)."""
    import clusterfusion as cf
    s, w, x, k, v, cos, sin = make_case("2b8", 17)
    w2 = dict(w)
    for n in ("ln_weight", "ln_bias", "post_ln_weight", "post_ln_bias"):
        w2[n] = w[n].reshape(1, -1)
    a = cf.pythia_2b8_decoder_layer(*layer_args(x, w, k.clone(), v.clone(), cos, sin, 17))
    b = cf.pythia_2b8_decoder_layer(*layer_args(x, w2, k.clone(), v.clone(), cos, sin, 17))
    assert torch.equal(a[0], b[0])


@pytest.mark.parametrize("model,seq", [("2b8", 257), ("6b9", 1000)])
def test_bitwise_deterministic(cuda_device, model, seq):
    """No atomics on data: 25 runs give identical bits (the reference's fp16 atomicAdd
    does not: tests/verify_lossless.py:229-246)."""
    s, w, x, k, v, cos, sin = make_case(model, seq)
    first = None
    for _ in range(25):
        out, kn, vn = fn_for(model)(*layer_args(x, w, k, v, cos, sin, seq))
        if first is None:
            first = (out.clone(), kn.clone(), vn.clone())
        else:
            assert torch.equal(out, first[0]) and torch.equal(kn, first[1]) and torch.equal(vn, first[2])


@pytest.mark.parametrize("model,seq", [("2b8", 0), ("2b8", 129), ("2b8", 1024), ("6b9", 777)])
def test_split_equals_fused_bitwise(cuda_device, model, seq):
    s, w, x, k, v, cos, sin = make_case(model, seq)
    k2, v2 = k.clone(), v.clone()
    a = fn_for(model)(*layer_args(x, w, k, v, cos, sin, seq))
    b = fn_for(model, split=True)(*layer_args(x, w, k2, v2, cos, sin, seq))
    for t, u in zip(a, b):
        assert torch.equal(t, u)
    assert torch.equal(k, k2) and torch.equal(v, v2)


@pytest.mark.parametrize("seq", [0, 129, 1024])
def test_attention_only_and_mlp_only(cuda_device, seq):
    """The two halves of the split API against the oracle's intermediates, and their
    composition against the fused op (fp16 hand-off between them, so not bitwise)."""
    import clusterfusion as cf
    s, w, x, k, v, cos, sin = make_case("2b8", seq)
    k0, v0 = k.clone(), v.clone()
    args = layer_args(x, w, k, v, cos, sin, seq)
    attn, mid, kn, vn = cf.pythia_2b8_attention_only(*args[:15], seq)
    assert attn.shape == (1, s.hidden) and mid.shape == (s.ffn,)
    inter = {}
    ro, rk, rv = O.layer_decode_fp32(s, x, w, k0, v0, cos, sin, seq, intermediates=inter)
    assert_close(attn, inter["attn_out"], "attn_output")
    assert_close(mid, inter["mid"], "mlp_intermediate")
    assert_close(kn, rk, "k_new")
    assert_close(vn, rv, "v_new")
    out = cf.pythia_2b8_mlp_only(x, attn, mid, w["mlp_down_weight"], w["mlp_down_bias"])
    assert_close(out, ro, "mlp_only output")
    fused, _, _ = cf.pythia_2b8_decoder_layer(*layer_args(x, w, k0.clone(), v0.clone(), cos, sin, seq))
    assert O.compare(out, fused.float())[0] <= 4e-3
    assert cf.device_status() == 0


def test_consecutive_steps_grow_the_cache(cuda_device):
    """Decode 6 positions in a row through one layer; every step must see the rows the
    previous steps appended (TMA reads of rows written by earlier launches)."""
    import clusterfusion as cf
    s = O.PYTHIA_2B8
    seq0, steps = 62, 6
    s, w, x, k, v, _, _ = make_case("2b8", seq0, rows=seq0 + steps + 1)
    cos_t, sin_t = O.rope_table(seq0 + steps + 1, s.rotary, device=x.device)
    kr, vr = k.clone().cpu().float(), v.clone().cpu().float()
    h = x
    hr = x.float().cpu()
    for i in range(steps):
        pos = seq0 + i
        out, kn, vn = cf.pythia_2b8_decoder_layer(*layer_args(h, w, k, v, cos_t[pos].contiguous(), sin_t[pos].contiguous(), pos))
        ro, rk, rv = O.layer_decode_fp32(s, hr, w, kr, vr, cos_t[pos], sin_t[pos], pos)
        assert_close(out, ro, f"step {i} output")
        kr[pos], vr[pos] = O.round_fp16(rk).reshape(-1), O.round_fp16(rv).reshape(-1)
        h = (out * 0.5).contiguous()       # keep magnitudes bounded without a final norm
        hr = h.float().cpu()


@pytest.mark.parametrize("bad", ["seq_too_large", "negative", "dtype", "noncontig", "shape", "cos_dtype"])
def test_argument_errors(cuda_device, bad):
    """Every misuse raises RuntimeError before anything is launched (the reference checks nothing)."""
    import clusterfusion as cf
    s, w, x, k, v, cos, sin = make_case("2b8", 10, rows=12)
    args = layer_args(x, w, k, v, cos, sin, 10)
    if bad == "seq_too_large":
        args[17] = 12          # no free row
    elif bad == "negative":
        args[17] = -1
    elif bad == "dtype":
        args[0] = x.float()
    elif bad == "noncontig":
        args[1] = w["qkv_weight"].t()
    elif bad == "shape":
        args[5] = k[:, :100].contiguous()
    elif bad == "cos_dtype":
        args[9] = cos.half()
    with pytest.raises(RuntimeError):
        cf.pythia_2b8_decoder_layer(*args)
    assert cf.device_status() == 0
