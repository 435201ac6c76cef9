"""Failure detection without a GPU fault: a tensor-parallel peer that never shows up.

A 2-rank decoder is built on ONE GPU and its "peer" exchange buffer is a zeroed buffer that
nothing ever writes, so the kernel's bounded wait for the peer's partial runs out (1.5 s).
The kernel must then finish by itself, report status 7 to the host, and leave the context
usable: the next, ordinary launch works.  Nothing traps, faults or hangs."""
import ctypes as C
import os
import sys
import time

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))
sys.path.insert(0, HERE)
import make_golden as G  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

pytestmark = pytest.mark.gpu


def test_missing_peer_times_out_and_is_reported(cuda_device):
    import clusterfusionplus_b200 as cf
    from clusterfusionplus_b200 import _lib
    from clusterfusionplus_b200.decoder import layer_weights_struct, rope_table
    dev = cuda_device
    s = O.Shape("tp-mini", hidden=1024, heads=8, head_dim=128, rotary=32, ffn=2048, vocab=1024, layers=2)
    full = cf.CfDims()
    full.hidden, full.heads, full.head_dim, full.rotary, full.ffn, full.vocab = (s.hidden, s.heads, s.head_dim, s.rotary,
                                                                                 s.ffn, s.vocab)
    d = cf.shard_dims(full, 2)
    layers = [cf.shard_layer_weights(O.make_layer_weights(s, l, seed=9, device=dev, std=0.05), full, 0, 2) for l in range(2)]
    head = cf.shard_head_weights(O.make_head_weights(s, seed=9, device=dev, std=0.05), full, 0, 2)
    max_seq = 8
    kvw = d.heads * d.head_dim
    caches = [(torch.zeros(max_seq, kvw, dtype=torch.float16, device=dev), torch.zeros(max_seq, kvw, dtype=torch.float16, device=dev))
              for _ in layers]
    cos, sin = rope_table(max_seq, s.rotary, dev)
    cfg = _lib.CfDecoderConfig()
    cfg.dims, cfg.n_layers, cfg.max_seq_len, cfg.tp_size, cfg.tp_rank = d, 2, max_seq, 2, 0
    cfg.cos_table, cfg.sin_table = cos.data_ptr(), sin.data_ptr()
    h = C.c_int64(0)
    _lib.check(_lib.lib.cf_decoder_create(C.byref(cfg), C.byref(h)))
    try:
        for i, (w, (k, v)) in enumerate(zip(layers, caches)):
            _lib.check(_lib.lib.cf_decoder_set_layer(h.value, i, C.byref(layer_weights_struct(d, w)), k.data_ptr(), v.data_ptr()))
        hw = _lib.CfHeadWeights()
        hw.embed_in, hw.final_ln_weight = head["embed_in"].data_ptr(), head["final_ln_weight"].data_ptr()
        hw.final_ln_bias, hw.embed_out, hw.vocab_offset = head["final_ln_bias"].data_ptr(), head["embed_out"].data_ptr(), 0
        _lib.check(_lib.lib.cf_decoder_set_head(h.value, C.byref(hw)))
        _lib.check(_lib.lib.cf_decoder_finalize(h.value))
        scratch = (C.c_char * 64)()
        _lib.check(_lib.lib.cf_decoder_tp_export(h.value, C.cast(scratch, C.c_void_p)))
        buf, nbytes = C.c_void_p(), C.c_int64(0)
        _lib.check(_lib.lib.cf_decoder_tp_buffer(h.value, C.byref(buf), C.byref(nbytes)))
        silent_peer = torch.zeros(nbytes.value + 256, dtype=torch.uint8, device=dev)   # rank 1 never writes here
        table = (C.c_void_p * 2)(buf.value, silent_peer.data_ptr())
        _lib.check(_lib.lib.cf_decoder_tp_connect_pointers(h.value, table))
        t0 = time.perf_counter()
        _lib.check(_lib.lib.cf_decoder_step(h.value, torch.cuda.current_stream().cuda_stream))
        with pytest.raises(RuntimeError, match="device status 7"):
            cf.device_status()
        waited = time.perf_counter() - t0
        assert 1.0 < waited < 10.0, waited          # one bounded wait, then everything else falls through
        assert cf.device_status() == 0               # status was cleared, barrier words re-armed
    finally:
        _lib.check(_lib.lib.cf_decoder_destroy(h.value))
    # the context is still healthy: an ordinary layer call gives the right answer
    from _util import assert_close, layer_args, make_case
    import clusterfusion
    s2, w, x, k, v, c, sn = make_case("2b8", 20)
    k0, v0 = k.clone(), v.clone()
    out, _, _ = clusterfusion.pythia_2b8_decoder_layer(*layer_args(x, w, k, v, c, sn, 20))
    ro, _, _ = O.layer_decode_fp32(s2, x, w, k0, v0, c, sn, 20)
    assert_close(out, ro, "layer after a timed-out launch")
    assert cf.device_status() == 0
