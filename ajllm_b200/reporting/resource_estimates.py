"""Memory and matrix-FLOP estimates for a training configuration.

Same result record as the reference (``ajllm/reporting/resource_estimates.py:11-106``) so that reports
and downstream tooling keep their fields; the model behind the numbers is generalised:

* projections count ``2 * tokens * D * (2 * Hq * hd + 2 * Hkv * hd)`` FLOPs (the reference counts
  ``10 * tokens * D^2`` for four ``D x D`` matrices, i.e. five of them; with full heads this estimate
  gives ``8 * tokens * D^2``);
* grouped KV heads, tied embeddings and mixture-of-experts layers (active parameters per token:
  ``top_k`` routed + shared experts + router) are understood;
* the two ``[B, H, T, T]`` attention matrices are only counted when ``flash_attention`` is false,
  since the tiled kernels never store them.

Training FLOPs are three forward equivalents; workspaces, fragmentation and non-matrix work are not
counted.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Any


@dataclass(frozen=True)
class ResourceEstimate:
    parameter_count: int
    parameter_bytes: int
    activation_elements: int
    activation_bytes: int
    gradient_bytes: int
    optimizer_bytes: int
    total_memory_bytes: int
    forward_flops_per_step: int
    training_flops_per_step: int
    total_training_flops: int
    total_training_steps: int
    total_training_tokens: int
    parameter_dtype_bytes: int
    activation_dtype_bytes: int
    optimizer_state_dtype_bytes: int


def _default_d_ff(d_model: int, kind: str) -> int:
    return ((int(8 * d_model / 3) + 63) // 64) * 64 if kind == "swiglu" else 4 * d_model


def estimate_resources(model_config: dict[str, Any], parameter_count: int, batch_size: int,
                       training_config: dict[str, Any] | None = None,
                       flash_attention: bool = False) -> ResourceEstimate:
    if batch_size < 1:
        raise ValueError("batch_size must be positive for resource estimation")
    training_config = training_config or {}
    T = int(model_config["context_length"])
    D = int(model_config["d_model"])
    L = int(model_config["num_layers"])
    Hq = int(model_config["num_heads"])
    Hkv = int(model_config.get("num_kv_heads", Hq))
    hd = D // Hq
    ff_kind = (model_config.get("feed_forward") or {}).get("type", "swiglu")
    F = int(model_config.get("d_ff", _default_d_ff(D, ff_kind)))
    V = int(model_config.get("vocab_size", training_config.get("vocab_size", 0)))
    if V < 1:
        V = int(model_config.get("report_vocab_size", 1))
    p_bytes = int(model_config.get("report_parameter_dtype_bytes", 4))
    a_bytes = int(model_config.get("report_activation_dtype_bytes", p_bytes))
    o_bytes = int(model_config.get("report_optimizer_state_dtype_bytes", 4))
    if min(p_bytes, a_bytes, o_bytes) < 1:
        raise ValueError("Resource dtype byte sizes must be positive")

    tokens = batch_size * T
    ffn_mats = 3 if ff_kind == "swiglu" else 2
    moe = model_config.get("moe") or None
    if moe:
        Fe = int(moe.get("d_ff", F))
        active = int(moe["top_k"]) + int(moe.get("shared_experts", 0))
        ffn_flops = 2 * tokens * D * (ffn_mats * Fe * active + int(moe["num_experts"]))
        ffn_saved = ffn_mats * tokens * Fe * active
    else:
        ffn_flops = ffn_mats * 2 * tokens * D * F
        ffn_saved = ffn_mats * tokens * F
    hidden = tokens * D
    attention_matrices = 0 if flash_attention else 2 * batch_size * Hq * T * T
    activation_elements = hidden + L * (5 * hidden + attention_matrices + ffn_saved) + tokens * V

    projection_flops = 2 * tokens * D * (2 * Hq * hd + 2 * Hkv * hd)
    attention_flops = 4 * batch_size * T * T * D
    forward = L * (projection_flops + attention_flops + ffn_flops) + 2 * tokens * D * V
    training = 3 * forward

    steps = int(training_config.get("max_steps", 0))
    if steps <= 0 and training_config.get("total_tokens") is not None:
        steps = max(1, math.ceil(int(training_config["total_tokens"]) / tokens))
    parameter_bytes = parameter_count * p_bytes
    activation_bytes = activation_elements * a_bytes
    gradient_bytes = parameter_count * p_bytes
    optimizer_bytes = parameter_count * 2 * o_bytes
    return ResourceEstimate(
        parameter_count=parameter_count, parameter_bytes=parameter_bytes,
        activation_elements=activation_elements, activation_bytes=activation_bytes,
        gradient_bytes=gradient_bytes, optimizer_bytes=optimizer_bytes,
        total_memory_bytes=parameter_bytes + activation_bytes + gradient_bytes + optimizer_bytes,
        forward_flops_per_step=forward, training_flops_per_step=training,
        total_training_flops=training * steps, total_training_steps=steps, total_training_tokens=steps * tokens,
        parameter_dtype_bytes=p_bytes, activation_dtype_bytes=a_bytes, optimizer_state_dtype_bytes=o_bytes,
    )
