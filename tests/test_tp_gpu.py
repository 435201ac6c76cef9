"""Tensor-parallel decode on 2, 4 and 8 GPUs of one box (one process per GPU, NCCL for set-up)
against the single-GPU decoder on identical seeded weights, Pythia-6.9B layer shapes with the
caches filled to 4096 rows (attention spans many chunks on every rank): hidden state within the
parity bar, greedy tokens identical on all ranks and equal to the single-GPU decoder's, CUDA-graph
replay bitwise equal to eager launches.  Each size is skipped on boxes with fewer GPUs."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

pytestmark = pytest.mark.gpu


def _worker(rank, size, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=size, device_id=dev)
    try:
        import clusterfusionplus_b200 as cf
        from oracle import pythia_oracle as O
        s = O.Shape("6b9-2l", 4096, 32, 128, 32, 16384, 50432, layers=2)
        full = cf.CfDims()
        full.hidden, full.heads, full.head_dim, full.rotary, full.ffn, full.vocab = 4096, 32, 128, 32, 16384, 50432
        layers = [O.make_layer_weights(s, l, seed=21, device=dev) for l in range(s.layers)]
        head = O.make_head_weights(s, seed=21, device=dev)
        ctx, steps = 4096, 6
        max_seq = ctx + steps + 2
        kv = [O.make_kv_cache(s, ctx, max_seq, 300 + l, device=dev) for l in range(s.layers)]
        loc_layers = [cf.shard_layer_weights(w, full, rank, size) for w in layers]
        loc_head = cf.shard_head_weights(head, full, rank, size)
        loc_kv = [(cf.shard_cache(k, full, rank, size), cf.shard_cache(v, full, rank, size)) for k, v in kv]
        tokens, hiddens = {}, {}
        # (fused in-kernel exchange, eager) / (fused, CUDA graph) / (NCCL all-reduce per layer, graph)
        for graph, fused in ((False, True), (True, True), ("nccl", False)):
            caches = [(k.clone(), v.clone()) for k, v in loc_kv]
            dec = cf.TPDecoder(full, loc_layers, loc_head, caches, max_seq, use_graph=bool(graph), fused=fused)
            dec.reset(ctx, 123)
            toks, hid = [], []
            for _ in range(steps):
                dec.step()
                toks.append(int(dec.token.item()))
                hid.append(dec.hidden.clone())
            assert int(dec.seq_len.item()) == ctx + steps
            tokens[graph], hiddens[graph] = toks, hid
            dec.close()
        assert tokens[False] == tokens[True] == tokens["nccl"]
        assert all(torch.equal(a, b) for a, b in zip(hiddens[False], hiddens[True]))   # graph replay == eager, bitwise
        for a, b in zip(hiddens[True], hiddens["nccl"]):                                # fp32 exchange vs fp16 NCCL wire
            assert O.compare(a, b)[0] <= 2e-2
        gathered = [None] * size
        dist.all_gather_object(gathered, tokens[True])
        assert all(g == gathered[0] for g in gathered), "ranks disagree on the tokens"
        if rank == 0:
            caches = [(k.clone(), v.clone()) for k, v in kv]
            ref = cf.PythiaDecoder(full, layers, head, caches, max_seq, use_graph=False)
            ref.reset(ctx, 123)
            ref_toks, errs = [], []
            for i in range(steps):
                ref.step()
                ref_toks.append(int(ref.token.item()))
                errs.append(O.compare(hiddens[True][i], ref.hidden))
            ref.close()
            ret["tokens"] = (tokens[True], ref_toks)
            ret["errs"] = errs
        ret[f"status{rank}"] = cf.device_status()
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("size", [2, 4, 8])
def test_tp_matches_single_gpu(cuda_device, size):
    if torch.cuda.device_count() < size:
        pytest.skip(f"needs {size} GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(size, 29731 + size, ret), nprocs=size, join=True)
    got, want = ret["tokens"]
    assert got == want
    for mx, rl in ret["errs"]:
        assert mx <= 2e-2 and rl <= 1e-3, (mx, rl)
    assert all(ret[f"status{r}"] == 0 for r in range(size))
