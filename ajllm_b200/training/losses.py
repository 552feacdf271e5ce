"""Training losses (reference: ``ajllm/training/losses.py:8-18``)."""

from __future__ import annotations

import torch

from ajllm_b200 import ops


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean cross-entropy over any leading dimensions; the reduction is fp32 whatever the logits dtype."""
    return ops.cross_entropy(logits, targets)
