"""HF GPT-NeoX state dict -> fused layout: checked on CPU by feeding the converted tensors to the
fp32 oracle and comparing its logits with the HuggingFace model the state dict came from."""
import pytest
import torch

from oracle import pythia_oracle as O


def tiny_neox(act: str, seed: int = 0):
    from transformers import GPTNeoXConfig, GPTNeoXForCausalLM
    cfg = GPTNeoXConfig(hidden_size=1024, num_attention_heads=8, intermediate_size=2048, num_hidden_layers=2,
                        vocab_size=1024, rotary_pct=0.25, hidden_act=act, max_position_embeddings=128,
                        use_parallel_residual=True, tie_word_embeddings=False)
    cfg._attn_implementation = "eager"
    torch.manual_seed(seed)
    model = GPTNeoXForCausalLM(cfg).float().eval()
    with torch.no_grad():  # both sides see exactly the fp16-representable weights
        for p in model.parameters():
            p.copy_(p.half().float())
            if p.ndim == 1:
                p.add_(torch.randn_like(p) * 0.02).copy_(p.half().float())  # biases / LN are not trivially 0 / 1
    return cfg, model


@pytest.mark.parametrize("act", ["gelu", "gelu_pytorch_tanh"])
def test_converted_state_dict_reproduces_hf_logits(act):
    import clusterfusionplus_b200 as cf
    cfg, model = tiny_neox(act)
    d, flags, base = cf.describe_config(cfg)
    assert (d.hidden, d.heads, d.head_dim, d.rotary, d.ffn, d.vocab) == (1024, 8, 128, 32, 2048, 1024)
    assert flags == (cf._lib.CF_DECODER_GELU_ERF if act == "gelu" else 0) and base == 10000.0
    layers, head = cf.convert_state_dict(model.state_dict(), cfg, device="cpu", dtype=torch.float32)
    shape = O.Shape("tiny", d.hidden, d.heads, d.head_dim, d.rotary, d.ffn, d.vocab, layers=2)
    om = O.OracleModel(shape, layers, head, max_seq=16, round_io=False, act="erf" if act == "gelu" else "tanh")
    ids = torch.randint(0, d.vocab, (1, 7), generator=torch.Generator().manual_seed(3))
    with torch.no_grad():
        ref = model(ids).logits[0]  # [7, V]
    for t in range(ids.shape[1]):
        logits, _ = om.step(int(ids[0, t]))
        assert torch.allclose(logits, ref[t], atol=2e-4, rtol=1e-4), (t, (logits - ref[t]).abs().max())


def test_unsupported_variants_are_refused():
    import clusterfusionplus_b200 as cf
    from transformers import GPTNeoXConfig
    base = dict(hidden_size=1024, num_attention_heads=8, intermediate_size=2048, num_hidden_layers=1, vocab_size=1024)
    with pytest.raises(RuntimeError):
        cf.describe_config(GPTNeoXConfig(**base, use_parallel_residual=False))
    with pytest.raises(RuntimeError):
        cf.describe_config(GPTNeoXConfig(**base, hidden_act="relu"))
    with pytest.raises(RuntimeError):
        cf.describe_config(GPTNeoXConfig(**base, layer_norm_eps=1e-6))


def test_quality_metric_definitions():
    """step_metrics / DecodeQuality on hand-made logits: the definitions of the reference's report
    (tests/evaluate_decode_quality.py:74-79, 161-199)."""
    import math
    from clusterfusionplus_b200.quality import DecodeQuality, kl_divergence, step_metrics
    ref = torch.arange(20, dtype=torch.float32)            # arg-max 19, top-5 = {15..19}
    same = ref.clone()
    m = step_metrics(ref, same, torch.ones(4), torch.ones(4))
    assert m == {"token_match": 1.0, "logits_mae": 0.0, "top5_agree": 1.0, "top10_agree": 1.0, "kl_divergence": 0.0,
                 "hidden_mae": 0.0}
    other = ref.clone()
    other[19], other[18] = ref[18], ref[19]               # swap the two best: token differs, the SETS agree
    m = step_metrics(ref, other)
    assert m["token_match"] == 0.0 and m["top5_agree"] == 1.0 and m["top10_agree"] == 1.0
    assert abs(m["logits_mae"] - 2.0 / 20) < 1e-7
    p, q = torch.tensor([0.0, math.log(3.0)]), torch.tensor([0.0, 0.0])   # p = (1/4, 3/4), q = (1/2, 1/2)
    assert abs(kl_divergence(p, q) - (0.25 * math.log(0.5) + 0.75 * math.log(1.5))) < 1e-6
    dq = DecodeQuality()
    dq.add(ref, same), dq.add(ref, other)
    s = dq.summary()
    assert s["total_tokens"] == 2 and s["token_match_rate"] == 50.0 and s["top5_agreement"] == 100.0
