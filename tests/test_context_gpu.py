"""create_graph_context / graph_decode_step / destroy_graph_context: the reference's
"CUDA graph" API (include/5090/pythia_6b9/pythia_kernel_dispatch_graph.cu), plus real
CUDA-graph capture and replay with device-resident sequence length."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _util import assert_close, layer_args, make_case, step_args  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def api(model):
    import clusterfusion as cf
    p = f"pythia_{model}_"
    return (getattr(cf, p + "create_graph_context"), getattr(cf, p + "graph_decode_step"),
            getattr(cf, p + "destroy_graph_context"), getattr(cf, p + "decoder_layer"),
            getattr(cf, p + "graph_set_device_state"))


@pytest.mark.parametrize("model,seq", [("2b8", 33), ("2b8", 1024), ("6b9", 129)])
def test_context_step_equals_eager_bitwise(cuda_device, model, seq):
    import clusterfusion as cf
    create, step, destroy, eager, _ = api(model)
    s, w, x, k, v, cos, sin = make_case(model, seq, rows=seq + 8)
    k2, v2 = k.clone(), v.clone()
    ref = eager(*layer_args(x, w, k2, v2, cos, sin, seq))
    create(5, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], seq + 8)
    try:
        out, kn, vn = step(*step_args(5, x, w, k, v, cos, sin, seq))
        assert out.shape == (1, s.hidden) and kn.shape == (1, s.heads, s.head_dim)
        for a, b in zip((out, kn, vn), ref):
            assert torch.equal(a, b)
        assert torch.equal(k, k2) and torch.equal(v, v2)
        # the returned tensors alias the context's static buffers
        # (pythia_kernel_dispatch_graph.cu:286 returns ctx.output itself)
        keep = out.clone()
        x2 = (x * 0.5).contiguous()
        out2, _, _ = step(*step_args(5, x2, w, k, v, cos, sin, seq))
        assert out2.data_ptr() == out.data_ptr()
        assert not torch.equal(keep, out2)
        ro, _, _ = O.layer_decode_fp32(s, x2, w, k2, v2, cos, sin, seq)
        assert_close(out2, ro, "second step")
    finally:
        destroy(5)
    assert cf.device_status() == 0


def test_unknown_context_raises(cuda_device):
    create, step, destroy, _, _ = api("2b8")
    s, w, x, k, v, cos, sin = make_case("2b8", 4)
    with pytest.raises(RuntimeError, match="Context not initialized"):
        step(*step_args(424242, x, w, k, v, cos, sin, 4))
    destroy(424242)  # erasing a missing id is not an error (map.erase in the reference)


def test_context_checks(cuda_device):
    create, step, destroy, _, _ = api("2b8")
    s, w, x, k, v, cos, sin = make_case("2b8", 4, rows=8)
    with pytest.raises(RuntimeError):
        create(1, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], 9)  # > rows
    create(1, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], 8)
    try:
        with pytest.raises(RuntimeError):
            step(*step_args(1, x, w, k, v, cos, sin, 8))            # no free row
        with pytest.raises(RuntimeError):
            step(*step_args(1, x, w, k.clone(), v, cos, sin, 4))    # not the context's cache
        out = step(*step_args(1, x, w, k, v, cos, sin, 4))[0].clone()
        # re-creating an id replaces it (and frees the old static buffers)
        create(1, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], 8)
        out2, _, _ = step(*step_args(1, x, w, k, v, cos, sin, 4))
        assert torch.equal(out, out2)
    finally:
        destroy(1)


def test_many_contexts_like_a_model(cuda_device):
    """One context per layer, keyed by layer index, as tests/benchmark_decode_6b9.py:118-131 does."""
    create, step, destroy, eager, _ = api("2b8")
    n = 4
    cases = [make_case("2b8", 20, rows=32, wseed=100 + i) for i in range(n)]
    for i, (s, w, x, k, v, cos, sin) in enumerate(cases):
        create(i, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], 32)
    try:
        h = cases[0][2]
        hr = h.clone()
        for i, (s, w, x, k, v, cos, sin) in enumerate(cases):
            k2, v2 = k.clone(), v.clone()
            h, _, _ = step(*step_args(i, h, w, k, v, cos, sin, 20))
            hr, _, _ = eager(*layer_args(hr, w, k2, v2, cos, sin, 20))
            h = h.clone()
        assert torch.equal(h, hr)
    finally:
        for i in range(n):
            destroy(i)


def test_programmatic_dependent_launch_chain_is_bitwise_identical(cuda_device, monkeypatch):
    """CFB200_PDL=1 chains the per-layer launches by programmatic dependent launch (each kernel streams its
    first weight stages while the one before it drains, and waits for it before touching anything else).
    Same bits as the plain chain, eagerly and inside a captured CUDA graph."""
    import clusterfusion as cf
    create, step, destroy, _, _ = api("2b8")
    n = 6
    cases = [make_case("2b8", 40, rows=48, wseed=300 + i) for i in range(n)]
    for i, (s, w, x, k, v, cos, sin) in enumerate(cases):
        create(20 + i, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], 48)
    snaps = [(c[3].clone(), c[4].clone()) for c in cases]
    x0 = cases[0][2].clone()

    def chain():
        h = x0
        for i, (s, w, x, k, v, cos, sin) in enumerate(cases):
            h, _, _ = step(*step_args(20 + i, h, w, k, v, cos, sin, 40))
        return h.clone()

    def restore():
        for (s, w, x, k, v, cos, sin), (ks, vs) in zip(cases, snaps):
            k.copy_(ks), v.copy_(vs)

    try:
        monkeypatch.setenv("CFB200_PDL", "0")
        plain = chain()
        torch.cuda.synchronize()
        restore()
        monkeypatch.setenv("CFB200_PDL", "1")
        for _ in range(3):
            got = chain()
            torch.cuda.synchronize()
            assert torch.equal(got, plain)
            restore()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = chain()
        for _ in range(3):
            restore()
            g.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, plain)
    finally:
        monkeypatch.setenv("CFB200_PDL", "0")
        for i in range(n):
            destroy(20 + i)
    assert cf.device_status() == 0


def test_real_cuda_graph_replay(cuda_device):
    """Capture graph_decode_step once with device-resident seq_len and RoPE table, then
    replay it for consecutive positions (the reference's mode cannot: it bakes seq_len
    into the launch, pythia_kernel_dispatch_graph.cu:260-261)."""
    import clusterfusion as cf
    create, step, destroy, eager, set_state = api("2b8")
    seq0, steps = 60, 8
    rows = seq0 + steps + 2
    s, w, x, k, v, _, _ = make_case("2b8", seq0, rows=rows)
    cos_t, sin_t = O.rope_table(rows, s.rotary, device=x.device)
    k_e, v_e = k.clone(), v.clone()
    seq_dev = torch.tensor([seq0], dtype=torch.int32, device=x.device)
    x_static = x.clone()
    create(9, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], rows)
    try:
        set_state(9, seq_dev, cos_t, sin_t)
        k_snap, v_snap = k.clone(), v.clone()
        out, kn, vn = step(*step_args(9, x_static, w, k, v, cos_t[0].contiguous(), sin_t[0].contiguous(), 0))  # uploads
        torch.cuda.synchronize()
        k.copy_(k_snap), v.copy_(v_snap)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step(*step_args(9, x_static, w, k, v, cos_t[0].contiguous(), sin_t[0].contiguous(), 0))
        k.copy_(k_snap), v.copy_(v_snap)
        h = x.clone()
        for i in range(steps):
            pos = seq0 + i
            seq_dev.fill_(pos)
            x_static.copy_(h)
            g.replay()
            ref, rk, rv = eager(*layer_args(h, w, k_e, v_e, cos_t[pos].contiguous(), sin_t[pos].contiguous(), pos))
            assert torch.equal(out, ref) and torch.equal(kn, rk) and torch.equal(vn, rv)
            h = (ref * 0.5).contiguous()
        assert torch.equal(k, k_e) and torch.equal(v, v_e)
    finally:
        destroy(9)
    assert cf.device_status() == 0


def test_bad_device_seq_len_is_reported_not_fatal(cuda_device):
    """A device-resident seq_len outside the cache makes the kernel return at once with
    a status word the host can read; the context stays usable."""
    import clusterfusion as cf
    create, step, destroy, eager, set_state = api("2b8")
    s, w, x, k, v, cos, sin = make_case("2b8", 4, rows=8)
    cos_t, sin_t = O.rope_table(8, s.rotary, device=x.device)
    seq_dev = torch.tensor([8], dtype=torch.int32, device=x.device)   # == rows: no free row
    create(3, k, v, w["qkv_weight"], w["o_weight"], w["mlp_up_weight"], w["mlp_down_weight"], 8)
    try:
        set_state(3, seq_dev, cos_t, sin_t)
        k0 = k.clone()
        step(*step_args(3, x, w, k, v, cos, sin, 0))
        with pytest.raises(RuntimeError, match="device status 5"):
            cf.device_status()
        assert torch.equal(k, k0)
        assert cf.device_status() == 0
        seq_dev.fill_(4)
        out, _, _ = step(*step_args(3, x, w, k, v, cos, sin, 0))
        ref, _, _ = eager(*layer_args(x, w, k0.clone(), v.clone(), cos_t[4].contiguous(), sin_t[4].contiguous(), 4))
        assert torch.equal(out, ref)
    finally:
        destroy(3)
