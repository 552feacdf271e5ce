"""Atomic checkpoints in the reference's dictionary layout (``ajllm/training/checkpoint.py:12-45``):
``{"model_state_dict", "optimizer_state_dict", "step", "metadata"}`` written to ``<path>.tmp`` and
renamed into place.

Model keys are always the un-sharded, un-prefixed reference names whatever the parallel layout (the
model's ``state_dict`` gathers tensor/expert-parallel shards; every rank must therefore enter
``save_checkpoint`` and only rank 0 touches the file system). Extra keys (``data_rng_state``,
``best_validation_loss``) ride in the same dictionary; the reference's loader ignores them.
"""

from __future__ import annotations

import os
import shutil
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist


def _is_writer() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def save_checkpoint(path: str | Path, model: torch.nn.Module, optimizer, step: int, metadata: dict[str, Any],
                    extra: dict[str, Any] | None = None, aliases: tuple[str, ...] = ()) -> Path:
    """Write ``path`` (and copies named ``aliases`` beside it, e.g. ``latest.pt``)."""
    target = Path(path)
    model_state = {k: v.detach().to("cpu") for k, v in model.state_dict().items()}
    optimizer_state = optimizer.state_dict() if optimizer is not None else None
    if not _is_writer():
        return target
    target.parent.mkdir(parents=True, exist_ok=True)
    payload = {
        "model_state_dict": model_state,
        "optimizer_state_dict": optimizer_state,
        "step": int(step),
        "metadata": metadata,
    }
    if extra:
        payload.update(extra)
    scratch = target.with_name(target.name + ".tmp")
    torch.save(payload, scratch)
    os.replace(scratch, target)
    for alias in aliases:
        alias_path = target.with_name(alias)
        alias_scratch = alias_path.with_name(alias_path.name + ".tmp")
        shutil.copyfile(target, alias_scratch)
        os.replace(alias_scratch, alias_path)
    return target


def load_checkpoint(path: str | Path, model: torch.nn.Module, optimizer=None,
                    map_location: str | torch.device = "cpu") -> dict[str, Any]:
    source = Path(path)
    try:
        checkpoint = torch.load(source, map_location="cpu", weights_only=False)
    except Exception as error:
        raise RuntimeError(f"Checkpoint {source} is unreadable (truncated or corrupt): {error}") from error
    for key in ("model_state_dict", "step"):
        if key not in checkpoint:
            raise RuntimeError(f"Checkpoint {source} has no '{key}' entry")
    state = checkpoint["model_state_dict"]
    # checkpoints written by the reference's FSDP wrapper carry a "module." prefix
    if state and all(key.startswith("module.") for key in state):
        state = {key[len("module."):]: value for key, value in state.items()}
    reference_dtype = next(model.parameters()).dtype
    state = {k: (v.to(reference_dtype) if torch.is_floating_point(v) else v) for k, v in state.items()}
    model.load_state_dict(state)
    if optimizer is not None and checkpoint.get("optimizer_state_dict") is not None:
        optimizer.load_state_dict(checkpoint["optimizer_state_dict"])
    return checkpoint
