"""The batched, paged Llama decode blocks (llama_decoder_layer_batch_decode_sglang and the batched SwiGLU MLP)
against the fp32 CPU oracle, through the C ABI: batch 1 / 4 / 16 (BASELINE config 5), up to 2048 cached rows per
sequence, ragged lengths (an empty history, one row, a chunk edge, the full 2048), page tables that scatter every
sequence over a shuffled pool, two layers' pools selected by layer_id.  The reference ships no test of this entry
point; the oracle's per-sequence arithmetic is the one pinned against transformers (oracle/llama_oracle.py)."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _util import MAX_ABS, REL_L2  # noqa: E402
from oracle import llama_oracle as LO  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu

H, NH, D, FFN = 4096, 32, 128, 11008
EPS = 1e-5


def cos_sin_table(n_pos, device):
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    ang = torch.outer(torch.arange(n_pos, dtype=torch.float32), inv)          # [pos, 64]
    return torch.cat([ang.cos(), ang.sin()], dim=1).contiguous().to(device)   # 64 cosines, then 64 sines


def make_pool_case(lengths, seed, dev):
    """Pools of two layers, a shuffled page table, inputs; history rows N(0,1) fp16."""
    B = len(lengths)
    g = torch.Generator().manual_seed(seed)
    n_rows = sum(lengths) + B + 37                                             # spare rows stay untouched
    perm = torch.randperm(n_rows, generator=g)
    indptr, indices, at = [0], [], 0
    for s in lengths:
        indices.append(perm[at:at + s + 1])                                    # history rows, then the new token's slot
        at += s + 1
        indptr.append(indptr[-1] + s + 1)
    pools = [(O.seeded_normal((n_rows, H), seed + 10 + 2 * l, device=dev), O.seeded_normal((n_rows, H), seed + 11 + 2 * l, device=dev))
             for l in range(2)]
    x = O.seeded_normal((B, H), seed + 1, device=dev)
    res = O.seeded_normal((B, H), seed + 2, device=dev)
    return dict(B=B, x=x, res=res, pools=pools,
                indptr=torch.tensor(indptr, dtype=torch.int32, device=dev),
                indices=torch.cat(indices).to(torch.int32).to(dev),
                positions=torch.tensor(lengths, dtype=torch.int64, device=dev))


@pytest.fixture(scope="module")
def weights(cuda_device):
    dev = cuda_device
    return dict(wqkv=O.seeded_normal((3 * H, H), 501, std=0.02, device=dev), wo=O.seeded_normal((H, H), 502, std=0.02, device=dev),
                g1=O.seeded_normal((H,), 503, mean=1.0, std=0.02, device=dev),
                wgu=O.seeded_normal((2 * FFN, H), 504, std=0.02, device=dev), wd=O.seeded_normal((H, FFN), 505, std=0.02, device=dev),
                g2=O.seeded_normal((H,), 506, mean=1.0, std=0.02, device=dev))


def close(got, ref, what):
    mx, rl = O.compare(got, ref)
    assert mx <= MAX_ABS and rl <= REL_L2, f"{what}: max-abs {mx:.3e} (<= {MAX_ABS}), rel-L2 {rl:.3e} (<= {REL_L2})"


@pytest.mark.parametrize("lengths", [
    [2048],                                                                     # batch 1
    [2048, 0, 129, 700],                                                        # batch 4, ragged, one empty history
    [2048, 2048, 2048, 2048],                                                   # batch 4 of config 5
    [2048, 1, 127, 128, 129, 2047, 0, 64, 1000, 1500, 300, 5, 2048, 777, 1024, 256],  # batch 16, ragged
], ids=["b1", "b4-ragged", "b4-2048", "b16-ragged"])
def test_attention_block_batch_vs_oracle(cuda_device, weights, lengths):
    import clusterfusion as cf
    dev = cuda_device
    c = make_pool_case(lengths, 900 + len(lengths), dev)
    layer = 1
    kp, vp = c["pools"][layer]
    k0, v0 = kp.clone(), vp.clone()
    other_k0 = c["pools"][0][0].clone()
    kptrs = torch.tensor([p[0].data_ptr() for p in c["pools"]], dtype=torch.int64, device=dev)
    vptrs = torch.tensor([p[1].data_ptr() for p in c["pools"]], dtype=torch.int64, device=dev)
    cs = cos_sin_table(2049, dev)
    out = torch.empty_like(c["x"])
    res_out = torch.empty_like(c["x"])
    ret = cf.llama_decoder_layer_batch_decode_sglang(out, res_out, c["x"], c["res"], weights["wqkv"], weights["wo"], c["indptr"],
                                                     c["indices"], kptrs, vptrs, layer, weights["g1"], EPS, c["positions"], cs)
    assert ret is None
    assert cf.device_status() == 0
    ro, rs, rk, rv, slots = LO.llama_attn_block_batch_fp32(c["x"], c["res"], weights["wqkv"], weights["wo"], k0, v0, c["indptr"],
                                                           c["indices"], c["positions"], cs, weights["g1"], EPS)
    close(out, ro, "output")
    assert torch.equal(res_out.cpu().float(), rs), "residual_output is input + residual rounded to fp16"
    close(kp[slots.to(dev)].view(-1, NH, D), rk, "appended keys")
    close(vp[slots.to(dev)].view(-1, NH, D), rv, "appended values")
    keep = torch.ones(kp.shape[0], dtype=torch.bool, device=dev)
    keep[slots.to(dev)] = False
    assert torch.equal(kp[keep], k0[keep]) and torch.equal(vp[keep], v0[keep]), "only the new tokens' slots are written"
    assert torch.equal(c["pools"][0][0], other_k0), "the other layer's pool is untouched"


@pytest.mark.parametrize("batch", [1, 4, 16])
def test_mlp_block_batch_vs_oracle(cuda_device, weights, batch):
    import clusterfusion as cf
    dev = cuda_device
    x = O.seeded_normal((batch, H), 71, device=dev)
    res = O.seeded_normal((batch, H), 72, device=dev)
    out, res_out = cf.llama_mlp_batch_sglang(x, res, weights["wgu"], weights["wd"], weights["g2"], EPS)
    assert cf.device_status() == 0
    ro, rs = LO.llama_mlp_block_batch_fp32(x, res, weights["wgu"], weights["wd"], weights["g2"], EPS)
    close(out, ro, "mlp output")
    assert torch.equal(res_out.cpu().float(), rs)


@pytest.mark.parametrize("ksplit", [1, 2])
def test_narrow_projections_without_and_with_two_k_slices(cuda_device, weights, ksplit, monkeypatch):
    """The down and output projections (28 rows per CTA) are cut along K over groups of CTAs by default (four
    slices, a reduction pass); CFB200_LB_KSPLIT selects the unsplit form (1) or two slices.  Same oracle bar."""
    import clusterfusion as cf
    dev = cuda_device
    monkeypatch.setenv("CFB200_LB_KSPLIT", str(ksplit))
    wd = weights["wd"].clone()          # new tensors: the tensor maps (and their slice count) are cached per tensor
    wo = weights["wo"].clone()
    x = O.seeded_normal((5, H), 81, device=dev)
    res = O.seeded_normal((5, H), 82, device=dev)
    out, res_out = cf.llama_mlp_batch_sglang(x, res, weights["wgu"], wd, weights["g2"], EPS)
    ro, rs = LO.llama_mlp_block_batch_fp32(x, res, weights["wgu"], wd, weights["g2"], EPS)
    close(out, ro, "mlp output")
    c = make_pool_case([300, 17, 2048], 77, dev)
    kptrs = torch.tensor([p[0].data_ptr() for p in c["pools"]], dtype=torch.int64, device=dev)
    vptrs = torch.tensor([p[1].data_ptr() for p in c["pools"]], dtype=torch.int64, device=dev)
    k0, v0 = c["pools"][0][0].clone(), c["pools"][0][1].clone()
    cs = cos_sin_table(2049, dev)
    o2, r2 = torch.empty_like(c["x"]), torch.empty_like(c["x"])
    cf.llama_decoder_layer_batch_decode_sglang(o2, r2, c["x"], c["res"], weights["wqkv"], wo, c["indptr"], c["indices"], kptrs, vptrs,
                                               0, weights["g1"], EPS, c["positions"], cs)
    ro2, _, _, _, _ = LO.llama_attn_block_batch_fp32(c["x"], c["res"], weights["wqkv"], wo, k0, v0, c["indptr"], c["indices"],
                                                     c["positions"], cs, weights["g1"], EPS)
    close(o2, ro2, "attention block output")
    assert cf.device_status() == 0


def test_batch_equals_batch1_block(cuda_device, weights):
    """The batched entry point at batch 1 against the batch-1 fused block (llama_decoder_layer_sglang) on the same
    sequence: same result within the parity bar (the two differ in where activations are rounded to fp16)."""
    import clusterfusion as cf
    dev = cuda_device
    c = make_pool_case([700], 4242, dev)
    kp, vp = c["pools"][0]
    rows = c["indices"][:700].long()
    kc, vc = kp[rows].contiguous(), vp[rows].contiguous()
    cs = cos_sin_table(1024, dev)
    cos = torch.cat([cs[700, :64], cs[700, :64]]).contiguous()
    sin = torch.cat([cs[700, 64:], cs[700, 64:]]).contiguous()
    o1, r1, k1, v1 = cf.llama_decoder_layer_sglang(c["x"].clone(), c["res"].clone(), weights["wqkv"], weights["wo"], kc, vc,
                                                   weights["g1"], EPS, cos, sin)
    out, res_out = torch.empty_like(c["x"]), torch.empty_like(c["x"])
    kptrs = torch.tensor([kp.data_ptr()], dtype=torch.int64, device=dev)
    vptrs = torch.tensor([vp.data_ptr()], dtype=torch.int64, device=dev)
    cf.llama_decoder_layer_batch_decode_sglang(out, res_out, c["x"], c["res"], weights["wqkv"], weights["wo"], c["indptr"],
                                               c["indices"], kptrs, vptrs, 0, weights["g1"], EPS, c["positions"], cs)
    assert cf.device_status() == 0
    close(out, o1, "batched vs batch-1 output")
    assert torch.equal(res_out, r1)
    slot = int(c["indices"][700])
    close(kp[slot].view(1, NH, D), k1, "appended key vs k_new")


def test_batch_argument_errors(cuda_device, weights):
    import clusterfusion as cf
    dev = cuda_device
    c = make_pool_case([5] * 17, 7, dev)
    kp, vp = c["pools"][0]
    kptrs = torch.tensor([kp.data_ptr()], dtype=torch.int64, device=dev)
    cs = cos_sin_table(16, dev)
    out, res_out = torch.empty_like(c["x"]), torch.empty_like(c["x"])
    with pytest.raises(RuntimeError, match="batch 17"):
        cf.llama_decoder_layer_batch_decode_sglang(out, res_out, c["x"], c["res"], weights["wqkv"], weights["wo"], c["indptr"],
                                                   c["indices"], kptrs, kptrs, 0, weights["g1"], EPS, c["positions"], cs)
    with pytest.raises(RuntimeError, match="layer_id"):
        cf.llama_decoder_layer_batch_decode_sglang(out[:4], res_out[:4], c["x"][:4], c["res"][:4], weights["wqkv"], weights["wo"],
                                                   c["indptr"][:5], c["indices"], kptrs, kptrs, 3, weights["g1"], EPS,
                                                   c["positions"][:4], cs)
