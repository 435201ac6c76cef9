"""Regenerates tests/golden/*.npz from the fp32 CPU oracle.

    python tests/golden/make_golden.py

Inputs are not stored (a 6.9B layer is 400 MB): every case is rebuilt from its
seed by oracle.pythia_oracle's generators, and the file carries float64 sums of
the regenerated tensors so a test can tell "inputs differ" from "outputs differ".
Outputs are the oracle's fp32 results.  The layer cases were cross-checked
against transformers' GPTNeoXLayer (oracle.pythia_oracle.hf_layer_decode) when
the files were made; HF_MAXDIFF records the largest difference seen.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
from oracle import llama_oracle as L  # noqa: E402
from oracle import pythia_oracle as O  # noqa: E402

# (name, model, seq_len, weight seed, input seed)
LAYER_CASES = [
    ("layer_2b8_seq33", "2b8", 33, 1234, 7),
    ("layer_2b8_seq0", "2b8", 0, 1234, 8),
    ("layer_2b8_seq1024", "2b8", 1024, 4321, 9),   # the single-layer benchmark configuration
    ("layer_6b9_seq129", "6b9", 129, 99, 10),      # sequence length of the reference's unit test
]

MINI = O.Shape("mini", hidden=512, heads=4, head_dim=128, rotary=32, ffn=2048, vocab=1024, layers=3)
# seed chosen so that the oracle's smallest top-2 logit gap over the rollout (0.026) is far
# above fp16 noise: greedy tokens are then a meaningful bit-exact check
MINI_ROLLOUT = dict(seed=14, prompt_len=5, steps=24)


def layer_case_inputs(model, seq_len, wseed, xseed, device="cpu"):
    s = O.SHAPES[model]
    w = O.make_layer_weights(s, 0, seed=wseed, device=device)
    x = O.seeded_normal((1, s.hidden), xseed, device=device)
    k, v = O.make_kv_cache(s, seq_len, seq_len + 3, xseed + 100, device=device)
    cos, sin = O.rope_table(seq_len + 1, s.rotary, device=device)
    return s, w, x, k, v, cos[seq_len].contiguous(), sin[seq_len].contiguous()


# Llama-2-7B blocks (hidden 4096, 32 heads x 128): (name, cached rows or ffn, seed)
LLAMA_ATTN_CASES = [("llama_attn_seq65", 65, 501), ("llama_attn_seq1", 1, 502)]
LLAMA_MLP_CASES = [("llama_mlp_ffn2048", 2048, 601), ("llama_mlp_ffn11008", 11008, 602)]
LLAMA_EPS = 1e-5


def llama_attn_inputs(seq, seed, device="cpu"):
    """fp16 tensors of one attention-block call, regenerated from the seed."""
    H, D = 4096, 128
    n = lambda shape, i, std, mean=0.0: O.seeded_normal(shape, seed + i, mean=mean, std=std, device=device).half()
    ang = torch.rand(D // 2, generator=torch.Generator().manual_seed(seed + 9)) * (2 * torch.pi)
    return dict(x=n((1, H), 0, 1.0), res=n((1, H), 1, 1.0), wqkv=n((3 * H, H), 2, 0.02), wo=n((H, H), 3, 0.02),
                k=n((seq, H), 4, 1.0), v=n((seq, H), 5, 1.0), g=n((1, H), 6, 0.1, 1.0),
                cos=torch.cat([ang.cos(), ang.cos()]).contiguous().to(device),
                sin=torch.cat([ang.sin(), ang.sin()]).contiguous().to(device))


def llama_mlp_inputs(ffn, seed, device="cpu"):
    H = 4096
    n = lambda shape, i, std, mean=0.0: O.seeded_normal(shape, seed + i, mean=mean, std=std, device=device).half()
    return dict(x=n((1, H), 0, 1.0), res=n((1, H), 1, 1.0), wgu=n((2 * ffn, H), 2, 0.02), wd=n((H, ffn), 3, 0.02),
                g=n((1, H), 4, 0.1, 1.0))


def checksum(*tensors):
    return np.array([t.double().sum().item() for t in tensors] + [t.double().abs().sum().item() for t in tensors])


def mini_model(device="cpu"):
    seed = MINI_ROLLOUT["seed"]
    layers = [O.make_layer_weights(MINI, l, seed=seed, device=device, std=0.05) for l in range(MINI.layers)]
    head = O.make_head_weights(MINI, seed=seed, device=device, std=0.05)
    return layers, head


def mini_rollout_oracle(round_io):
    layers, head = mini_model()
    cfg = MINI_ROLLOUT
    max_seq = cfg["prompt_len"] + cfg["steps"] + 2
    om = O.OracleModel(MINI, layers, head, max_seq, round_io=round_io)
    g = torch.Generator().manual_seed(cfg["seed"])
    prompt = torch.randint(0, MINI.vocab, (cfg["prompt_len"],), generator=g).tolist()
    logits = None
    for t in prompt:
        logits, _ = om.step(t)
    tok = int(logits.argmax())
    tokens, gaps = [], []
    for _ in range(cfg["steps"]):
        tokens.append(tok)
        logits, _ = om.step(tok)
        top2 = torch.topk(logits, 2).values
        gaps.append((top2[0] - top2[1]).item())
        tok = int(logits.argmax())
    return prompt, tokens, gaps, logits


def main():
    for name, model, seq, wseed, xseed in LAYER_CASES:
        s, w, x, k, v, cos, sin = layer_case_inputs(model, seq, wseed, xseed)
        out, kn, vn = O.layer_decode_fp32(s, x, w, k, v, cos, sin, seq)
        ho, hk, hv = O.hf_layer_decode(s, x, w, k, v, seq, seq)
        hf = max(O.compare(out, ho)[0], O.compare(kn, hk)[0], O.compare(vn, hv)[0])
        assert hf < 2e-5, (name, hf)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), out=out.numpy(), k_new=kn.numpy(), v_new=vn.numpy(),
                            in_checksum=checksum(x, w["qkv_weight"], w["mlp_down_weight"], k, v), hf_maxdiff=np.array(hf))
        print(name, "hf maxdiff", hf)
    for name, seq, seed in LLAMA_ATTN_CASES:
        t = llama_attn_inputs(seq, seed)
        args = (t["x"], t["res"], t["wqkv"], t["wo"], t["k"], t["v"], t["g"], LLAMA_EPS, t["cos"], t["sin"])
        out, res, kn, vn = L.llama_attn_block_fp32(*args)
        ho, hr, hk, hv = L.hf_llama_attn_block(*args)
        hf = max(O.compare(out, ho)[0], O.compare(kn, hk)[0], O.compare(vn, hv)[0])
        assert hf < 2e-5 and torch.equal(res, hr), (name, hf)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), out=out.numpy(), residual=res.numpy(), k_new=kn.numpy(),
                            v_new=vn.numpy(), in_checksum=checksum(t["x"], t["wqkv"], t["wo"], t["k"], t["v"]),
                            hf_maxdiff=np.array(hf))
        print(name, "hf maxdiff", hf)
    for name, ffn, seed in LLAMA_MLP_CASES:
        t = llama_mlp_inputs(ffn, seed)
        args = (t["x"], t["res"], t["wgu"], t["wd"], t["g"], LLAMA_EPS)
        out, res = L.llama_mlp_block_fp32(*args)
        ho, hr = L.hf_llama_mlp_block(*args)
        hf = O.compare(out, ho)[0]
        assert hf < 2e-5 and torch.equal(res, hr), (name, hf)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), out=out.numpy(), residual=res.numpy(),
                            in_checksum=checksum(t["x"], t["wgu"], t["wd"]), hf_maxdiff=np.array(hf))
        print(name, "hf maxdiff", hf)
    prompt, tokens, gaps, logits = mini_rollout_oracle(round_io=False)
    np.savez_compressed(os.path.join(HERE, "mini_rollout.npz"), prompt=np.array(prompt), tokens=np.array(tokens),
                        gaps=np.array(gaps), last_logits=logits.numpy())
    print("mini rollout tokens", tokens, "min top-2 gap", min(gaps))


if __name__ == "__main__":
    main()
