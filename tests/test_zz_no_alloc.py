"""The allocation-free layer entry point (cf_pythia_decoder_layer_noalloc), called
through the C ABI with caller-owned buffers, against the regular entry point.

Who needs it: code that cannot allocate device memory where it calls the layer --
an inference server whose memory pool has already reserved all of HBM (a late
cudaMalloc would fail or fragment the pool), or a caller that sits inside its own
allocator's critical section.  Such callers hand in inputs and outputs only; the
kernel's scratch is a static device array inside the library.

Collected last on purpose (file name): a failure here cannot hide the other tests
from a run that stops at the first failure.  Works alone in a fresh process too.
"""
import ctypes as C
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from _util import make_case  # noqa: E402

pytestmark = pytest.mark.gpu


def _structs(model, s, w, x, k, v, cos, sin, out, kn, vn):
    from clusterfusionplus_b200 import _lib, api, model_dims
    d = model_dims(model)
    ws = api._weights(d, w["qkv_weight"], w["qkv_bias"], w["o_weight"], w["o_bias"], w["ln_weight"], w["ln_bias"],
                      w["post_ln_weight"], w["post_ln_bias"], w["mlp_up_weight"], w["mlp_up_bias"],
                      w["mlp_down_weight"], w["mlp_down_bias"])
    io = _lib.CfLayerIO()
    io.input, io.k_cache, io.v_cache, io.kv_rows = x.data_ptr(), k.data_ptr(), v.data_ptr(), k.shape[0]
    io.cos, io.sin = cos.data_ptr(), sin.data_ptr()
    io.output, io.k_new, io.v_new = out.data_ptr(), kn.data_ptr(), vn.data_ptr()
    return ws, io


def _call(entry, model_id, name, seq, x, w, k, v, cos, sin, s):
    """One call of a C entry point with buffers the caller (this test) owns."""
    from clusterfusionplus_b200 import _lib
    dev = x.device
    out = torch.empty((1, s.hidden), dtype=torch.float16, device=dev)
    kn = torch.empty((1, s.heads, s.head_dim), dtype=torch.float16, device=dev)
    vn = torch.empty_like(kn)
    ws, io = _structs(model_id, s, w, x, k, v, cos, sin, out, kn, vn)
    _lib.check(entry(model_id, C.byref(ws), C.byref(io), seq, torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return out, kn, vn


@pytest.mark.parametrize("model", ["2b8", "6b9"])
def test_noalloc_matches_regular_entry_point_twice(cuda_device, model):
    """Two calls in a row (the second sees the row the first appended, a new input, and the
    static array still holding the first call's contents): outputs, new K/V and the cache
    rows must equal the regular entry point's bit for bit -- it is the same kernel with the
    same reduction order, only its scratch lives elsewhere."""
    import clusterfusionplus_b200 as cf
    from clusterfusionplus_b200 import _lib
    from oracle import pythia_oracle as O
    model_id = cf.CF_PYTHIA_2B8 if model == "2b8" else cf.CF_PYTHIA_6B9
    seq = 70
    s, w, x, k, v, _, _ = make_case(model, seq, rows=seq + 4)
    cos_t, sin_t = O.rope_table(seq + 4, s.rotary, device=x.device)
    k_ref, v_ref = k.clone(), v.clone()
    x2 = O.seeded_normal((1, s.hidden), 4711, device=x.device)
    for step, xin in enumerate((x, x2)):
        pos = seq + step
        c, sn = cos_t[pos].contiguous(), sin_t[pos].contiguous()
        got = _call(_lib.lib.cf_pythia_decoder_layer_noalloc, model_id, "noalloc", pos, xin, w, k, v, c, sn, s)
        ref = _call(_lib.lib.cf_pythia_decoder_layer, model_id, "regular", pos, xin, w, k_ref, v_ref, c, sn, s)
        for name, a, b in zip(("output", "k_new", "v_new"), got, ref):
            assert torch.equal(a, b), f"call {step + 1}: {name} differs from the regular entry point"
        assert torch.equal(k, k_ref) and torch.equal(v, v_ref), f"call {step + 1}: cache rows differ"
    assert cf.device_status() == 0


def test_noalloc_device_status_is_reported(cuda_device):
    """A device-side failure of a noalloc launch must reach the host.  The failure is made on the
    host: a status code is copied into the static array's status word (what a kernel whose bounded
    wait ran out would have left there); nothing on the GPU is made to wait or fault.  The next
    noalloc call must not wipe it, cf_get_status must report it and clear it."""
    import clusterfusionplus_b200 as cf
    from clusterfusionplus_b200 import _lib
    from clusterfusionplus_b200.decoder import _IntView
    base, nbytes, off = C.c_void_p(), C.c_int64(0), C.c_int64(0)
    _lib.check(_lib.lib.cf_debug_noalloc_scratch(C.byref(base), C.byref(nbytes), C.byref(off)))
    assert base.value and 0 < off.value < nbytes.value
    word = torch.as_tensor(_IntView(base.value + off.value, (1,)), device=cuda_device)
    assert cf.device_status() == 0
    word.fill_(3)                                   # "a flag wait ran out"
    torch.cuda.synchronize()
    s, w, x, k, v, cos, sin = make_case("2b8", 5, rows=7)
    _call(_lib.lib.cf_pythia_decoder_layer_noalloc, cf.CF_PYTHIA_2B8, "noalloc", 5, x, w, k, v, cos, sin, s)
    assert int(word.item()) == 3                    # the call left the earlier failure readable
    with pytest.raises(RuntimeError, match="device status 3"):
        cf.device_status()
    assert int(word.item()) == 0 and cf.device_status() == 0


def test_noalloc_new_tensors_refused_during_capture(cuda_device):
    """A call whose tensors differ from the previous call's uploads a new descriptor from host memory;
    recorded into a stream capture that copy would read a dead pointer at every replay, so the entry
    point refuses it while the stream is capturing.  Nothing is launched or replayed here."""
    import clusterfusionplus_b200 as cf
    from clusterfusionplus_b200 import _lib
    s, w, x, k, v, cos, sin = make_case("2b8", 5, rows=7, wseed=99)
    _call(_lib.lib.cf_pythia_decoder_layer_noalloc, cf.CF_PYTHIA_2B8, "noalloc", 5, x, w, k, v, cos, sin, s)
    k2, v2 = k.clone(), v.clone()                   # a tensor set the descriptor slot does not hold
    out = torch.empty((1, s.hidden), dtype=torch.float16, device=x.device)
    kn = torch.empty((1, s.heads, s.head_dim), dtype=torch.float16, device=x.device)
    vn = torch.empty_like(kn)
    ws, io = _structs(cf.CF_PYTHIA_2B8, s, w, x, k2, v2, cos, sin, out, kn, vn)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        g.capture_begin()
        try:
            rc = _lib.lib.cf_pythia_decoder_layer_noalloc(cf.CF_PYTHIA_2B8, C.byref(ws), C.byref(io), 5, side.cuda_stream)
            msg = _lib.last_error()
        finally:
            g.capture_end()
    assert rc != 0 and "capture" in msg, (rc, msg)
    del g
    torch.cuda.synchronize()
    assert cf.device_status() == 0


def test_noalloc_argument_errors(cuda_device):
    """Same argument checks as the regular entry point: no free cache row -> error, nothing launched."""
    import clusterfusionplus_b200 as cf
    from clusterfusionplus_b200 import _lib
    s, w, x, k, v, cos, sin = make_case("2b8", 5, rows=6)
    with pytest.raises(RuntimeError, match="current_seq_len"):
        _call(_lib.lib.cf_pythia_decoder_layer_noalloc, cf.CF_PYTHIA_2B8, "noalloc", 6, x, w, k, v, cos, sin, s)
    out = _call(_lib.lib.cf_pythia_decoder_layer_noalloc, cf.CF_PYTHIA_2B8, "noalloc", 5, x, w, k, v, cos, sin, s)
    assert torch.isfinite(out[0].float()).all()
