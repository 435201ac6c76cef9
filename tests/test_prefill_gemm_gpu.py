"""Tensor-core prefill linear (cf_prefill_linear) against a plain PyTorch fp32 reference of the
same op: act(x W^T + bias + residual), fp16 operands, fp32 accumulation, fp16 result."""
import pytest
import torch
import torch.nn.functional as F

from tests._util import MAX_ABS, REL_L2

pytestmark = pytest.mark.gpu


def _ref(x, w, b, r, act):
    y = x.float() @ w.float().t()
    if b is not None:
        y = y + b.float()
    if r is not None:
        y = y + r.float()
    if act == 1:
        y = F.gelu(y, approximate="tanh")
    elif act == 2:
        y = F.gelu(y)
    return y


@pytest.mark.parametrize("m,n,k", [(1, 1024, 1024), (7, 3072, 1024), (100, 2048, 1024), (511, 4096, 4096),
                                   (1024, 16384, 4096), (129, 2560, 10240), (300, 7680, 2560)])
@pytest.mark.parametrize("act", [0, 1, 2])
def test_prefill_linear_matches_fp32_reference(m, n, k, act):
    from clusterfusionplus_b200.decoder import prefill_linear
    g = torch.Generator(device="cuda").manual_seed(m * 7 + n + k + act)
    x = torch.randn(m, k, device="cuda", generator=g).half()
    w = (torch.randn(n, k, device="cuda", generator=g) * 0.02).half()
    b = (torch.randn(n, device="cuda", generator=g) * 0.02).half()
    r = torch.randn(m, n, device="cuda", generator=g).half() if act == 0 else None
    for bias, res in ((b, r), (None, None)):
        out = prefill_linear(x, w, bias, res, act)
        ref = _ref(x, w, bias, res, act)
        err = (out.float() - ref).abs().max().item()
        rel = ((out.float() - ref).norm() / ref.norm()).item()
        assert err <= MAX_ABS and rel <= REL_L2, (err, rel)


def test_prefill_linear_rejects_bad_arguments():
    from clusterfusionplus_b200.decoder import prefill_linear
    x = torch.zeros(4, 1024, device="cuda", dtype=torch.half)
    w = torch.zeros(1020, 1024, device="cuda", dtype=torch.half)
    with pytest.raises(RuntimeError):
        prefill_linear(x, w)  # n not a multiple of 8
    w = torch.zeros(1024, 1024, device="cuda", dtype=torch.half)
    with pytest.raises(RuntimeError):
        prefill_linear(x, w, residual=torch.zeros(4, 1024, device="cuda", dtype=torch.half), act=1)


@pytest.mark.parametrize("m,hidden", [(1, 4096), (37, 2560), (300, 4096), (5, 1024)])
def test_prefill_layernorm2_vs_torch(m, hidden):
    """Both LayerNorms of a block in one pass (cf_prefill_layernorm2) against torch's fp32 layer_norm."""
    from clusterfusionplus_b200 import _lib
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(m * 7 + hidden)
    x = (torch.randn(m, hidden, generator=g, device=dev) * 1.5 + 0.3).half()
    ws = [(torch.randn(hidden, generator=g, device=dev) * 0.1 + (1.0 if i % 2 == 0 else 0.0)).half() for i in range(4)]
    y1, y2 = torch.empty_like(x), torch.empty_like(x)
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.cf_prefill_layernorm2(x.data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(), ws[2].data_ptr(), ws[3].data_ptr(),
                                              y1.data_ptr(), y2.data_ptr(), m, hidden, 1e-5, st))
    r1 = torch.nn.functional.layer_norm(x.float(), (hidden,), ws[0].float(), ws[1].float(), 1e-5)
    r2 = torch.nn.functional.layer_norm(x.float(), (hidden,), ws[2].float(), ws[3].float(), 1e-5)
    assert (y1.float() - r1).abs().max().item() <= 4e-3 and (y2.float() - r2).abs().max().item() <= 4e-3
    # second output optional
    y3 = torch.empty_like(x)
    _lib.check(_lib.lib.cf_prefill_layernorm2(x.data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(), None, None, y3.data_ptr(), None, m,
                                              hidden, 1e-5, st))
    assert torch.equal(y3, y1)
    assert _lib.lib.cf_prefill_layernorm2(x.data_ptr(), ws[0].data_ptr(), ws[1].data_ptr(), None, None, y3.data_ptr(), None, m,
                                          hidden + 4, 1e-5, st) != 0


@pytest.mark.parametrize("heads,head_dim,rotary,m", [(32, 128, 32, 33), (32, 80, 20, 7), (8, 128, 128, 64), (4, 128, 0, 3)])
def test_prefill_rope_split_vs_torch(heads, head_dim, rotary, m):
    """Rotated queries, rotated keys and values into cache rows (cf_prefill_rope_split) against the torch expression
    the prompt pass used before (rotate-half in fp32, rounded to fp16)."""
    from clusterfusionplus_b200 import _lib
    import clusterfusionplus_b200 as cf
    dev = "cuda:0"
    g = torch.Generator(device=dev).manual_seed(heads + m)
    qkv = torch.randn(m, heads, 3, head_dim, generator=g, device=dev).half()
    rows = m + 5
    kvw = heads * head_dim
    kc = torch.full((rows, kvw), 7.0, device=dev, dtype=torch.float16)
    vc = torch.full((rows, kvw), 7.0, device=dev, dtype=torch.float16)
    q = torch.empty(m, heads, head_dim, device=dev, dtype=torch.float16)
    cos, sin = cf.rope_table(rows, rotary, dev) if rotary else (torch.zeros(rows, 1, device=dev), torch.zeros(rows, 1, device=dev))
    st = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.cf_prefill_rope_split(qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), q.data_ptr(), kc.data_ptr(),
                                              vc.data_ptr(), m, heads, head_dim, rotary, kvw, st))

    def rope(t):
        if rotary == 0:
            return t
        r = t[..., :rotary].float()
        c, s = cos[:m, None, :], sin[:m, None, :]
        half = torch.cat([-r[..., rotary // 2:], r[..., : rotary // 2]], dim=-1)
        return torch.cat([(r * c + half * s).to(t.dtype), t[..., rotary:]], dim=-1)

    assert (q.float() - rope(qkv[:, :, 0]).float()).abs().max().item() <= 2e-3
    assert (kc[:m].view(m, heads, head_dim).float() - rope(qkv[:, :, 1]).float()).abs().max().item() <= 2e-3
    assert torch.equal(vc[:m].view(m, heads, head_dim), qkv[:, :, 2])
    assert torch.all(kc[m:] == 7.0) and torch.all(vc[m:] == 7.0)      # rows beyond the prompt untouched
