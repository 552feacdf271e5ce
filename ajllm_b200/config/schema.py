"""Validation of resolved configs.

The required keys and consistency rules of the reference (``ajllm/config/validation.py:10-33``) are
kept; the checks for grouped-query attention, mixture-of-experts and the parallel mesh are
extensions that default to the reference's behaviour when the keys are absent.
"""

from __future__ import annotations

from typing import Any

from ajllm_b200.config.loader import ConfigError


def require(mapping: dict[str, Any], keys: tuple[str, ...], what: str) -> None:
    absent = [key for key in keys if key not in mapping]
    if absent:
        raise ConfigError(f"Missing {what} configuration values: {', '.join(absent)}")


def check_dataset(dataset: dict[str, Any]) -> None:
    require(dataset, ("name", "splits"), "dataset")
    splits = dataset["splits"]
    if not isinstance(splits, dict) or not splits:
        raise ConfigError("dataset.splits must be a non-empty mapping")


def check_tokenizer(tokenizer: dict[str, Any]) -> None:
    require(tokenizer, ("name", "vocab_size"), "tokenizer")
    floor = 256 + len(tokenizer.get("special_tokens", []) or [])
    if int(tokenizer["vocab_size"]) < floor:
        raise ConfigError("tokenizer.vocab_size is too small for all bytes and special tokens")


def check_model(model: dict[str, Any]) -> None:
    require(model, ("name", "context_length", "d_model", "num_layers", "num_heads"), "model")
    d_model, heads = int(model["d_model"]), int(model["num_heads"])
    if heads <= 0 or d_model % heads != 0:
        raise ConfigError("model.d_model must be divisible by model.num_heads")
    if int(model["context_length"]) < 2:
        raise ConfigError("model.context_length must be at least 2")
    kv_heads = int(model.get("num_kv_heads", heads))
    if kv_heads <= 0 or heads % kv_heads != 0:
        raise ConfigError("model.num_kv_heads must divide model.num_heads")
    moe = model.get("moe")
    if moe:
        require(moe, ("num_experts", "top_k"), "model.moe")
        if not 0 < int(moe["top_k"]) <= int(moe["num_experts"]):
            raise ConfigError("model.moe.top_k must be in [1, num_experts]")


def check_parallel(parallel: dict[str, Any], world_size: int) -> dict[str, int]:
    """Return the mesh extents ``{tp, ep, fsdp, pp, cp}``; their product (EP shares FSDP's ranks) must fill
    the world. Context parallelism (``cp``) takes the innermost axis in place of ``tp`` and combines with
    replicated data parallelism only."""
    tp = int(parallel.get("tp", 1))
    pp = int(parallel.get("pp", 1))
    ep = int(parallel.get("ep", 1))
    cp = int(parallel.get("cp", 1))
    fsdp = int(parallel.get("fsdp", max(1, world_size // (tp * pp * cp))))
    if min(tp, pp, ep, fsdp, cp) < 1:
        raise ConfigError("parallel extents must be positive")
    if cp > 1 and (tp > 1 or pp > 1 or ep > 1):
        raise ConfigError("parallel.cp combines with data parallelism only (tp = pp = ep = 1)")
    if tp * pp * fsdp * cp != world_size:
        raise ConfigError(f"parallel.tp*pp*fsdp*cp = {tp * pp * fsdp * cp} does not match world size {world_size}")
    if fsdp % ep != 0 and ep % fsdp != 0:
        raise ConfigError("parallel.ep must divide, or be a multiple of, parallel.fsdp")
    return {"tp": tp, "ep": ep, "fsdp": fsdp, "pp": pp, "cp": cp}
