"""Speculative decoding: acceptance rule and bookkeeping.

A small draft model proposes ``k`` tokens ``d_1..d_k`` with distributions ``q_1..q_k``; the target
model scores all ``k+1`` positions in one pass, giving ``p_1..p_{k+1}``. Token ``d_i`` is accepted
with probability ``min(1, p_i(d_i) / q_i(d_i))``; at the first rejection a replacement is drawn from
``normalise(max(0, p_i - q_i))`` and the step ends; if every draft token is accepted a bonus token is
drawn from ``p_{k+1}``. The emitted tokens are distributed exactly as samples from the target model.
With temperature 0 both distributions are one-hot, which reduces the rule to "accept while the draft
token equals the target argmax, then emit the target argmax". The reference has no speculative decoding.
"""

from __future__ import annotations

import torch


def verify_greedy(draft_tokens: torch.Tensor, target_logits: torch.Tensor) -> tuple[int, int]:
    """``draft_tokens [k]``, ``target_logits [k+1, vocab]`` -> ``(accepted, next_token)``."""
    best = torch.argmax(target_logits, dim=-1)
    k = draft_tokens.shape[0]
    accepted = 0
    while accepted < k and int(draft_tokens[accepted]) == int(best[accepted]):
        accepted += 1
    return accepted, int(best[accepted])


def verify_rejection(draft_tokens: torch.Tensor, draft_probs: torch.Tensor, target_probs: torch.Tensor,
                     generator: torch.Generator | None = None) -> tuple[int, int]:
    """``draft_probs [k, vocab]`` (the distributions the draft tokens were drawn from),
    ``target_probs [k+1, vocab]`` -> ``(accepted, next_token)``."""
    k = draft_tokens.shape[0]
    uniforms = torch.rand(k, generator=generator, device="cpu")
    for i in range(k):
        token = int(draft_tokens[i])
        p, q = float(target_probs[i, token]), float(draft_probs[i, token])
        if q > 0 and float(uniforms[i]) * q <= p:
            continue
        residual = torch.clamp(target_probs[i].float() - draft_probs[i].float(), min=0.0)
        mass = float(residual.sum())
        if mass <= 0:                     # p == q everywhere: any sample from p is a valid correction
            residual, mass = target_probs[i].float(), float(target_probs[i].sum())
        pick = torch.multinomial((residual / mass).cpu(), 1, generator=generator)
        return i, int(pick)
    pick = torch.multinomial(target_probs[k].float().cpu(), 1, generator=generator)
    return k, int(pick)
