"""Autoregressive generation with the reference's call signature
(``ajllm/generation/generator.py:10-28``), served by the paged-KV engine instead of re-running the
model on the whole context for every token."""

from __future__ import annotations

import torch

from ajllm_b200.engine.engine import LLMEngine
from ajllm_b200.engine.scheduler import SamplingParams


@torch.no_grad()
def generate(model: torch.nn.Module, prompt_tokens: torch.Tensor, max_new_tokens: int, temperature: float = 1.0,
             top_p: float | None = None, eos_token_id: int | None = None, seed: int | None = None) -> torch.Tensor:
    """Returns prompt + generated tokens as a 1-D tensor; stops after ``eos_token_id`` (inclusive)."""
    prompt = [int(t) for t in prompt_tokens.reshape(-1).tolist()]
    # the reference slides its window over the last context_length tokens; a cache cannot slide, so the
    # total length is capped at the model's context instead
    budget = max(0, min(max_new_tokens, model.context_length + 1 - len(prompt)))
    if budget == 0:
        return prompt_tokens.reshape(-1)
    engine = LLMEngine(model, block_size=16, max_num_seqs=1, max_batched_tokens=max(len(prompt), 16),
                       seed=seed if seed is not None else int(torch.initial_seed() % (2**31)))
    out = engine.generate([prompt], SamplingParams(budget, temperature, top_p, eos_token_id, seed))[0]
    return torch.tensor(prompt + out.output, dtype=prompt_tokens.dtype, device=prompt_tokens.device)
