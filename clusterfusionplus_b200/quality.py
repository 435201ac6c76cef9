"""Decode-quality metrics of the fused decoder against a reference model, step by step.

The metric set of the reference's tests/evaluate_decode_quality.py:74-79,131-199: both sides are fed the
REFERENCE's token at every step (teacher forcing, :149-150), and per step the harness records whether the
arg-max tokens agree, the mean absolute error of the logits (and of the final hidden state when both are
given), whether the top-5 and top-10 token SETS agree, and KL(reference || decoder) of the softmax
distributions; the summary reports rates in percent and means, under the reference's key names.

The reference runs this on downloaded Pythia checkpoints and English prompts; neither is available offline,
so the tests run it on a random-init model of the same architecture (what the metrics measure -- numerical
agreement of two implementations on the same weights -- does not depend on the weights being trained).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn.functional as F


def kl_divergence(ref_logits: torch.Tensor, got_logits: torch.Tensor, temperature: float = 1.0) -> float:
    """KL(softmax(ref) || softmax(got)), natural log (compute_kl_divergence of the reference, :74-79)."""
    p = F.log_softmax(ref_logits.float().reshape(-1) / temperature, dim=-1)
    q = F.log_softmax(got_logits.float().reshape(-1) / temperature, dim=-1)
    return float((p.exp() * (p - q)).sum())


def step_metrics(ref_logits: torch.Tensor, got_logits: torch.Tensor, ref_hidden: Optional[torch.Tensor] = None,
                 got_hidden: Optional[torch.Tensor] = None) -> Dict[str, float]:
    r, g = ref_logits.float().reshape(-1).cpu(), got_logits.float().reshape(-1).cpu()
    rt, gt = torch.topk(r, 10).indices.tolist(), torch.topk(g, 10).indices.tolist()
    out = {
        "token_match": float(int(r.argmax()) == int(g.argmax())),
        "logits_mae": float((r - g).abs().mean()),
        "top5_agree": float(set(rt[:5]) == set(gt[:5])),
        "top10_agree": float(set(rt) == set(gt)),
        "kl_divergence": kl_divergence(r, g),
    }
    if ref_hidden is not None and got_hidden is not None:
        out["hidden_mae"] = float((ref_hidden.float().reshape(-1).cpu() - got_hidden.float().reshape(-1).cpu()).abs().mean())
    return out


class DecodeQuality:
    """Accumulates step_metrics(); summary() has the reference's keys (rates in percent)."""

    def __init__(self):
        self.steps: List[Dict[str, float]] = []

    def add(self, *args, **kw) -> Dict[str, float]:
        m = step_metrics(*args, **kw)
        self.steps.append(m)
        return m

    def summary(self) -> Dict[str, float]:
        n = len(self.steps)
        if n == 0:
            raise RuntimeError("no steps recorded")
        mean = lambda k: sum(s[k] for s in self.steps if k in s) / max(1, sum(1 for s in self.steps if k in s))
        out = {"total_tokens": n, "token_match_rate": 100.0 * mean("token_match"), "logits_mae": mean("logits_mae"),
               "top5_agreement": 100.0 * mean("top5_agree"), "top10_agreement": 100.0 * mean("top10_agree"),
               "kl_divergence": mean("kl_divergence")}
        if any("hidden_mae" in s for s in self.steps):
            out["hidden_mae"] = mean("hidden_mae")
        return out


def evaluate_decode_quality(decoder, reference_step: Callable[[int], Tuple[torch.Tensor, Optional[torch.Tensor]]],
                            first_token: int, n_tokens: int) -> Dict[str, float]:
    """Teacher-forced comparison over n_tokens decode steps.

    decoder        : a positioned PythiaDecoder (prefill() or reset() done); its step() consumes decoder.token
    reference_step : token id -> (logits [vocab], final hidden state [hidden] or None) of the reference model,
                     which keeps its own cache (e.g. a HuggingFace model with past_key_values, or the fp32 oracle)
    The reference's arg-max token is fed to both sides at the next step, as the reference script does."""
    q = DecodeQuality()
    tok = int(first_token)
    for _ in range(n_tokens):
        ref_logits, ref_hidden = reference_step(tok)
        decoder.token.fill_(tok)
        decoder.step()
        q.add(ref_logits, decoder.logits, ref_hidden, decoder.hidden if ref_hidden is not None else None)
        tok = int(ref_logits.float().reshape(-1).argmax())
    return q.summary()
