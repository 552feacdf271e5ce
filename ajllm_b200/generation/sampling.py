"""Next-token sampling (reference: ``ajllm/generation/sampling.py:8-22``).

``temperature <= 0`` is greedy argmax. Otherwise ``softmax(logits / T)``; with ``top_p < 1`` the
tokens are sorted by probability and a token is kept when the cumulative mass *before* it is still
below ``top_p`` (so the token that crosses the threshold is kept), the kept mass is renormalised and
one token is drawn. The batched form takes per-row temperature / top-p and an optional per-row
generator so that a request's samples do not depend on which other requests share its batch.
"""

from __future__ import annotations

import torch

from ajllm_b200.ops import reference


def sampling_probabilities(logits: torch.Tensor, temperature: float, top_p: float | None) -> torch.Tensor:
    """The distribution ``sample_next_token`` draws from (rows of ``logits``), as fp32 probabilities."""
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    if top_p is not None and top_p < 1.0:
        probs = reference.top_p_filter(probs, top_p)
    return probs


def sample_next_token(logits: torch.Tensor, temperature: float, top_p: float | None,
                      generator: torch.Generator | None = None) -> torch.Tensor:
    """``logits`` is ``[rows, vocab]``; returns ``[rows, 1]`` token ids."""
    if temperature <= 0:
        return torch.argmax(logits, dim=-1, keepdim=True)
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    if top_p is not None and top_p < 1.0:
        if not 0 < top_p <= 1:
            raise ValueError("top_p must be in (0, 1]")
        # draw in sorted order, as the reference does, so equal seeds give equal tokens
        ordered, index = torch.sort(probs, descending=True, dim=-1)
        before = torch.cumsum(ordered, dim=-1) - ordered
        ordered = ordered.masked_fill(before >= top_p, 0.0)
        ordered = ordered / ordered.sum(dim=-1, keepdim=True)
        return torch.gather(index, -1, torch.multinomial(ordered, 1, generator=generator))
    return torch.multinomial(probs, 1, generator=generator)


def sample_batch(logits: torch.Tensor, temperatures: list[float], top_ps: list[float | None],
                 generators: list[torch.Generator | None] | None = None) -> torch.Tensor:
    """Row ``i`` is sampled with its own ``(temperature, top_p, generator)``; returns ``[rows]`` ids."""
    rows = logits.shape[0]
    out = torch.empty(rows, dtype=torch.long, device=logits.device)
    greedy = [i for i in range(rows) if temperatures[i] <= 0]
    if greedy:
        idx = torch.tensor(greedy, device=logits.device)
        out[idx] = torch.argmax(logits[idx], dim=-1)
    for i in range(rows):
        if temperatures[i] <= 0:
            continue
        gen = generators[i] if generators is not None else None
        out[i] = sample_next_token(logits[i:i + 1], temperatures[i], top_ps[i], gen)[0, 0]
    return out
