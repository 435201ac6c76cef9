"""Tensor-parallel partition checked on the CPU with two gloo ranks: each rank runs the
oracle on its shard (heads + MLP columns), the fp16 partials are all-reduced, and the
finished layer must equal the unsharded oracle.  This is the host-side contract the GPU
path implements (shard helpers in clusterfusionplus_b200/tp.py)."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))


def _worker(rank, size, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=size)
    try:
        import make_golden as G
        from clusterfusionplus_b200 import CfDims, shard_cache, shard_dims, shard_head_weights, shard_layer_weights
        from oracle import pythia_oracle as O
        s = G.MINI
        full = CfDims()
        full.hidden, full.heads, full.head_dim, full.rotary, full.ffn, full.vocab = (s.hidden, s.heads, s.head_dim,
                                                                                     s.rotary, s.ffn, s.vocab)
        d = shard_dims(full, size)
        assert (d.heads, d.ffn, d.vocab, d.hidden) == (s.heads // size, s.ffn // size, s.vocab // size, s.hidden)
        seq = 37
        w = O.make_layer_weights(s, 0, seed=3, std=0.05)
        head = O.make_head_weights(s, seed=3, std=0.05)
        x = O.seeded_normal((1, s.hidden), 4)
        k, v = O.make_kv_cache(s, seq, seq + 2, 5)
        cos, sin = O.rope_table(seq + 1, s.rotary)
        ws = shard_layer_weights(w, full, rank, size)
        ks, vs = shard_cache(k, full, rank, size), shard_cache(v, full, rank, size)
        local = O.Shape("shard", s.hidden, d.heads, s.head_dim, s.rotary, d.ffn, d.vocab)
        part, kn, vn = O.layer_decode_fp32(local, x, ws, ks, vs, cos[seq], sin[seq], seq, partial=True)
        part = part.half().float()              # the wire format of the per-layer all-reduce is fp16
        dist.all_reduce(part)
        out = x.float() + part + w["o_bias"].float() + w["mlp_down_bias"].float()
        ref, rk, rv = O.layer_decode_fp32(s, x, w, k, v, cos[seq], sin[seq], seq)
        err_out = O.compare(out, ref)
        nh = d.heads
        err_k = O.compare(kn, rk[:, rank * nh:(rank + 1) * nh])
        err_v = O.compare(vn, rv[:, rank * nh:(rank + 1) * nh])
        # vocabulary-sharded arg-max: every rank must pick the global winner
        hs = shard_head_weights(head, full, rank, size)
        lg = O.final_logits_fp32(ref, hs).reshape(-1)
        mine = torch.tensor([lg.max().item(), float(lg.argmax().item() + rank * d.vocab)])
        allp = [torch.zeros(2) for _ in range(size)]
        dist.all_gather(allp, mine)
        best = max(allp, key=lambda t: (t[0].item(), -t[1].item()))
        full_arg = int(O.final_logits_fp32(ref, head).reshape(-1).argmax())
        ret[rank] = (err_out, err_k, err_v, int(best[1].item()) == full_arg)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("size", [2, 4])
def test_tp_partition_matches_unsharded_oracle(size):
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29600 + size
    mp.spawn(_worker, args=(size, port, ret), nprocs=size, join=True)
    assert len(ret) == size
    for rank in range(size):
        err_out, err_k, err_v, arg_ok = ret[rank]
        assert err_out[0] < 2e-2 and err_out[1] < 1e-3, err_out  # fp16 wire format of the partials
        assert err_k[0] < 1e-5 and err_v[0] < 1e-5
        assert arg_ok
