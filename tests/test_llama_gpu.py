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
