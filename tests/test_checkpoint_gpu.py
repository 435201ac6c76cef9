"""End to end against HuggingFace: a small random GPTNeoXForCausalLM is converted with the
checkpoint adaptor, its prompt is ingested by prefill() and the fused kernel continues greedily;
tokens must equal HF's own greedy generation in fp32 on the CPU."""
import pytest
import torch

from tests._util import MAX_ABS
from tests.test_checkpoint_cpu import tiny_neox

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("act", ["gelu", "gelu_pytorch_tanh"])
def test_hf_checkpoint_prefill_and_greedy_decode(act):
    import clusterfusionplus_b200 as cf
    cfg, model = tiny_neox(act, seed=1)
    n_new = 24
    prompt = torch.randint(0, cfg.vocab_size, (1, 9), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        ref = model.generate(prompt, max_new_tokens=n_new, do_sample=False, pad_token_id=0)[0, prompt.shape[1]:].tolist()
        full = torch.cat([prompt[0], torch.tensor(ref)])[None]
        ref_logits = model(full).logits[0]  # row t = logits after consuming token t
    dec = cf.load_decoder(model.state_dict(), cfg, max_seq=64, device="cuda:0", use_graph=False)
    # teacher-forced: same inputs on both sides, logits within the parity tolerance at every step
    dec.prefill(prompt[0].tolist())
    worst = 0.0
    for t in range(n_new):
        pos = prompt.shape[1] - 1 + t
        dec.token.fill_(int(full[0, pos]))
        dec.step()
        err = (dec.logits.float().cpu() - ref_logits[pos]).abs().max().item()
        worst = max(worst, err)
    assert worst <= MAX_ABS, worst
    # free-running greedy generation: identical tokens
    got = dec.generate_from_prompt(prompt[0].tolist(), n_new)
    top2 = ref_logits[prompt.shape[1] - 1:-1].topk(2, dim=-1).values
    assert got == ref, (got, ref, (top2[:, 0] - top2[:, 1]).min().item())
    assert cf.device_status() == 0
    dec.close()


def test_prefill_fills_the_caches_like_token_by_token_decode():
    """prefill() (library GEMMs over all positions) and feeding the prompt one token at a time
    through the fused kernel must leave the same cache rows, within fp16 tolerance."""
    import clusterfusionplus_b200 as cf
    cfg, model = tiny_neox("gelu_pytorch_tanh", seed=2)
    prompt = torch.randint(0, cfg.vocab_size, (12,), generator=torch.Generator().manual_seed(7)).tolist()
    a = cf.load_decoder(model.state_dict(), cfg, max_seq=32, device="cuda:0", use_graph=False)
    b = cf.load_decoder(model.state_dict(), cfg, max_seq=32, device="cuda:0", use_graph=False)
    a.prefill(prompt)
    b.reset(0, prompt[0])
    for t in range(len(prompt) - 1):
        b.token.fill_(prompt[t])
        b.step()
    torch.cuda.synchronize()
    m = len(prompt) - 1
    for (ka, va), (kb, vb) in zip(a.caches, b.caches):
        assert (ka[:m].float() - kb[:m].float()).abs().max().item() <= MAX_ABS
        assert (va[:m].float() - vb[:m].float()).abs().max().item() <= MAX_ABS
    assert int(a.seq_len.item()) == m and int(a.token.item()) == prompt[-1]
    a.close()
    b.close()


def test_decode_quality_metrics_against_huggingface():
    """The reference's decode-quality report (tests/evaluate_decode_quality.py:131-199: token match, logits MAE,
    top-5 / top-10 agreement, KL divergence, teacher forced) between HuggingFace in fp32 and the fused decoder,
    on a random-init model of the architecture (no checkpoint is available offline)."""
    import clusterfusionplus_b200 as cf
    cfg, model = tiny_neox("gelu", seed=3)
    prompt = torch.randint(0, cfg.vocab_size, (1, 11), generator=torch.Generator().manual_seed(9))
    n_new = 32
    state = {}
    with torch.no_grad():
        out = model(prompt[:, :-1], use_cache=True)
        state["past"] = out.past_key_values

    def hf_step(token):
        with torch.no_grad():
            o = model(torch.tensor([[token]]), past_key_values=state["past"], use_cache=True, output_hidden_states=True)
        state["past"] = o.past_key_values
        return o.logits[0, -1], None

    dec = cf.load_decoder(model.state_dict(), cfg, max_seq=64, device="cuda:0", use_graph=False)
    dec.prefill(prompt[0].tolist())
    rep = cf.evaluate_decode_quality(dec, hf_step, int(prompt[0, -1]), n_new)
    assert rep["total_tokens"] == n_new
    assert rep["token_match_rate"] == 100.0 and rep["top5_agreement"] >= 95.0, rep
    assert rep["logits_mae"] <= 2e-3 and rep["kl_divergence"] <= 1e-5, rep
    assert cf.device_status() == 0
    dec.close()
