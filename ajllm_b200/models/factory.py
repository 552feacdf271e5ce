"""Build a model from a resolved ``model:`` mapping (reference: ``ajllm/modeling/factory.py:11-35``).

Defaults are the reference's: RoPE with theta 1e4, pre-norm RMSNorm, SwiGLU with
``d_ff = 64 * ceil((8/3 d_model) / 64)`` (``4 d_model`` for the SiLU FFN), untied head. Added keys:
``num_kv_heads``, ``init: {type, std}``, ``moe: {...}``, ``norm_epsilon``.
"""

from __future__ import annotations

from typing import Any

from ajllm_b200.config.schema import check_model
from ajllm_b200.models.layers import InitSpec
from ajllm_b200.models.transformer import TransformerLM


def default_d_ff(d_model: int, feed_forward: str) -> int:
    if feed_forward == "swiglu":
        return ((int(8 * d_model / 3) + 63) // 64) * 64
    return 4 * d_model


def build_model(config: dict[str, Any], vocab_size: int, use_flash_attention: bool = False, *,
                tp=None, ep=None, activation_checkpointing: str = "none", cp=None) -> TransformerLM:
    """``use_flash_attention`` is accepted for config compatibility; attention is always the tiled
    kernel on a GPU and the exact softmax on the CPU."""
    check_model(config)
    position = config.get("position_encoding") or {}
    normalization = config.get("normalization") or {}
    feed_forward = config.get("feed_forward") or {}
    d_model = int(config["d_model"])
    ff_type = str(feed_forward.get("type", "swiglu"))
    moe = config.get("moe") or None
    if moe:
        moe = dict(moe)
        moe.setdefault("d_ff", int(config.get("d_ff", default_d_ff(d_model, ff_type))))
    return TransformerLM(
        vocab_size=vocab_size,
        context_length=int(config["context_length"]),
        d_model=d_model,
        num_layers=int(config["num_layers"]),
        num_heads=int(config["num_heads"]),
        num_kv_heads=int(config.get("num_kv_heads", config["num_heads"])),
        d_ff=int(config.get("d_ff", default_d_ff(d_model, ff_type))),
        position_encoding=str(position.get("type", "rope")),
        rope_theta=float(position.get("theta", 10_000.0)),
        normalization=str(normalization.get("type", "rmsnorm")),
        norm_placement=str(normalization.get("placement", "pre")),
        feed_forward=ff_type,
        tie_embeddings=bool(config.get("tie_embeddings", False)),
        moe=moe,
        init=InitSpec.from_config(config.get("init")),
        tp=tp,
        ep=ep,
        cp=cp,
        norm_epsilon=float(config.get("norm_epsilon", 1e-5)),
        activation_checkpointing=activation_checkpointing,
    )


def count_parameters(config: dict[str, Any], vocab_size: int) -> int:
    """Closed-form parameter count (dense: ``2VD + L(…)+D`` as in the reference README, generalised to
    grouped KV heads, tied heads and MoE)."""
    d = int(config["d_model"])
    layers = int(config["num_layers"])
    heads = int(config["num_heads"])
    kv = int(config.get("num_kv_heads", heads))
    hd = d // heads
    ff_type = str((config.get("feed_forward") or {}).get("type", "swiglu"))
    f = int(config.get("d_ff", default_d_ff(d, ff_type)))
    norm = (config.get("normalization") or {}).get("type", "rmsnorm") == "rmsnorm"
    placement = (config.get("normalization") or {}).get("placement", "pre")
    attn = d * heads * hd * 2 + 2 * d * kv * hd
    moe = config.get("moe")
    if moe:
        fe = int(moe.get("d_ff", f))
        ffn = int(moe["num_experts"]) * 3 * d * fe + int(moe.get("shared_experts", 0)) * 3 * d * fe \
            + int(moe["num_experts"]) * d
    else:
        ffn = (3 if ff_type == "swiglu" else 2) * d * f
    per_layer = attn + ffn + (2 * d if norm else 0)
    total = vocab_size * d + layers * per_layer
    if not config.get("tie_embeddings", False):
        total += vocab_size * d
    if norm and placement == "pre":
        total += d
    if (config.get("position_encoding") or {}).get("type", "rope") == "learned":
        total += int(config["context_length"]) * d
    return total
