"""Helpers shared by workflows that consume a finished training run
(reference: ``ajllm/workflows/common.py:15-53``)."""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch
import yaml

from ajllm_b200.models import build_model
from ajllm_b200.training.checkpoint import load_checkpoint

CHECKPOINT_ALIASES = ("best", "latest", "final")


def project_path(project_root: Path, value: str | Path) -> Path:
    path = Path(value)
    return path if path.is_absolute() else (project_root / path).resolve()


def load_run_configuration(run_directory: Path) -> dict[str, Any]:
    with (run_directory / "resolved_config.yaml").open("r", encoding="utf-8") as handle:
        return yaml.safe_load(handle)


def select_checkpoint(run_directory: Path, selector: str) -> Path:
    """``best`` / ``latest`` / ``final``, a path relative to the run directory, or a ``.pt`` file."""
    direct = Path(selector)
    if direct.suffix == ".pt" and direct.is_file():
        return direct
    if selector in CHECKPOINT_ALIASES:
        candidate = run_directory / "checkpoints" / f"{selector}.pt"
    else:
        candidate = run_directory / selector
    if not candidate.is_file():
        raise FileNotFoundError(f"Checkpoint does not exist: {candidate}")
    return candidate


def inference_dtype(device: torch.device, run_config: dict[str, Any]) -> torch.dtype:
    """bf16 on a GPU (the kernels' native type), fp32 on the CPU."""
    return torch.bfloat16 if device.type == "cuda" else torch.float32


def load_model_from_run(run_directory: Path, checkpoint_selector: str, device: torch.device, tp=None
                        ) -> tuple[torch.nn.Module, dict[str, Any], dict[str, Any]]:
    """``tp`` (a :class:`~ajllm_b200.parallel.TensorParallel`) makes every rank load its own slice of the
    un-sharded checkpoint."""
    run_config = load_run_configuration(run_directory)
    vocab_size = int(run_config["_runtime"]["vocab_size"])
    model = build_model(run_config["model"], vocab_size, tp=tp).to(device=device, dtype=inference_dtype(device, run_config))
    checkpoint = load_checkpoint(select_checkpoint(run_directory, checkpoint_selector), model)
    model.eval()
    return model, run_config, checkpoint


def dump_yaml(path: Path, data: dict[str, Any]) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with path.open("w", encoding="utf-8") as handle:
        yaml.safe_dump(data, handle, sort_keys=False, allow_unicode=True)
