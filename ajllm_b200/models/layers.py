"""Parameter-holding building blocks.

Shapes, the bias-free convention and the default initialisation follow the reference
(``ajllm/modeling/layers.py:9-82``): ``Linear.weight`` is ``[out, in]`` with truncated-normal
``std = sqrt(2 / (in + out))`` clipped at three sigma; ``Embedding.weight`` is ``[rows, dim]`` with
truncated-normal ``std = 1`` clipped at +-3; ``RMSNorm.weight`` starts at one. ``init`` may instead ask
for plain ``normal`` with a fixed ``std`` (used by the large benchmark configurations).
"""

from __future__ import annotations

from dataclasses import dataclass

import torch
from torch import nn

from ajllm_b200 import ops


@dataclass(frozen=True)
class InitSpec:
    kind: str = "reference"      # "reference" | "normal"
    std: float = 0.02

    @staticmethod
    def from_config(config: dict | None) -> "InitSpec":
        config = config or {}
        return InitSpec(str(config.get("type", "reference")), float(config.get("std", 0.02)))


def init_matrix_(weight: torch.Tensor, fan_in: int, fan_out: int, spec: InitSpec) -> None:
    if spec.kind == "normal":
        nn.init.normal_(weight, mean=0.0, std=spec.std)
    elif spec.kind == "reference":
        std = (2.0 / (fan_in + fan_out)) ** 0.5
        nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
    else:
        raise ValueError(f"Unsupported init type: {spec.kind}")


def init_embedding_(weight: torch.Tensor, spec: InitSpec) -> None:
    if spec.kind == "normal":
        nn.init.normal_(weight, mean=0.0, std=spec.std)
    else:
        nn.init.trunc_normal_(weight, mean=0.0, std=1.0, a=-3.0, b=3.0)


class Linear(nn.Module):
    def __init__(self, in_features: int, out_features: int, init: InitSpec = InitSpec(),
                 device=None, dtype=None) -> None:
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.weight = nn.Parameter(torch.empty(out_features, in_features, device=device, dtype=dtype))
        init_matrix_(self.weight.data, in_features, out_features, init)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight)

    def extra_repr(self) -> str:
        return f"in={self.in_features}, out={self.out_features}"


class Embedding(nn.Module):
    def __init__(self, num_embeddings: int, embedding_dim: int, init: InitSpec = InitSpec(),
                 device=None, dtype=None) -> None:
        super().__init__()
        self.num_embeddings, self.embedding_dim = num_embeddings, embedding_dim
        self.weight = nn.Parameter(torch.empty(num_embeddings, embedding_dim, device=device, dtype=dtype))
        init_embedding_(self.weight.data, init)

    def forward(self, ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(ids, self.weight)


class RMSNorm(nn.Module):
    def __init__(self, d_model: int, epsilon: float = 1e-5, device=None, dtype=None) -> None:
        super().__init__()
        self.epsilon = epsilon
        self.weight = nn.Parameter(torch.ones(d_model, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.rms_norm(x, self.weight, self.epsilon)

    def add_and_norm(self, x: torch.Tensor, delta: torch.Tensor | None):
        """``(x + delta, norm(x + delta))`` in one pass over the activations."""
        return ops.add_rms_norm(x, delta, self.weight, self.epsilon)


class NoNorm(nn.Module):
    """Stand-in for ``normalization.type: none``."""

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def add_and_norm(self, x: torch.Tensor, delta: torch.Tensor | None):
        h = x if delta is None else x + delta
        return h, h


def make_norm(kind: str, d_model: int, epsilon: float = 1e-5) -> nn.Module:
    if kind == "rmsnorm":
        return RMSNorm(d_model, epsilon)
    if kind == "none":
        return NoNorm()
    raise ValueError(f"Unsupported normalization type: {kind}")
