"""Seed every random source a run touches (reference: ``ajllm/utils/random.py:11-16``)."""

from __future__ import annotations

import random

import numpy as np
import torch


def seed_all(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed % (2**32))
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)
