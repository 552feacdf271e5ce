"""Learning-rate schedule (reference: ``ajllm/training/schedulers.py:8-22``).

Linear warm-up from zero over ``warmup_steps``, half-cosine from ``max_lr`` down to ``min_lr`` at
``total_steps``, flat ``min_lr`` afterwards.
"""

from __future__ import annotations

import math


def warmup_cosine_learning_rate(step: int, max_learning_rate: float, min_learning_rate: float,
                                warmup_steps: int, total_steps: int) -> float:
    if 0 < warmup_steps and step < warmup_steps:
        return max_learning_rate * (step / warmup_steps)
    if step >= total_steps:
        return min_learning_rate
    span = max(1, total_steps - warmup_steps)
    phase = math.pi * (step - warmup_steps) / span
    return min_learning_rate + 0.5 * (1.0 + math.cos(phase)) * (max_learning_rate - min_learning_rate)
