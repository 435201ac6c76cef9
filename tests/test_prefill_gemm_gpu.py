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
