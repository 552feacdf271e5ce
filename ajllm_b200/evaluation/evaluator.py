"""Loss / perplexity of a model over random held-out batches
(reference: ``ajllm/evaluation/evaluator.py:14-31``; result keys ``loss``, ``perplexity``, ``batches``)."""

from __future__ import annotations

import math

import numpy as np
import torch


@torch.no_grad()
def evaluate_model(model: torch.nn.Module, dataset, batches: int, batch_size: int, context_length: int,
                   device: torch.device, seed: int) -> dict[str, float]:
    was_training = model.training
    model.eval()
    generator = np.random.default_rng(seed)
    running = torch.zeros((), dtype=torch.float64, device=device)
    for _ in range(batches):
        inputs, targets = dataset.batch(batch_size, context_length, device, generator)
        running += model.loss(inputs, targets).double()      # stays on the device; one read-back at the end
    if was_training:
        model.train()
    loss = float(running.item()) / batches
    return {"loss": loss, "perplexity": math.exp(min(loss, 50.0)), "batches": batches}
