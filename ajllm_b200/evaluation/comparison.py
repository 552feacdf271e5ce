"""Rank completed runs by a ``summary.json`` metric (reference: ``ajllm/evaluation/comparison.py:12-33``)."""

from __future__ import annotations

import csv
import json
from pathlib import Path
from typing import Any


def load_run_summary(run_directory: str | Path) -> dict[str, Any]:
    folder = Path(run_directory)
    with (folder / "summary.json").open("r", encoding="utf-8") as handle:
        summary = json.load(handle)
    return {"run_directory": str(folder.resolve()), **summary}


def compare_runs(run_directories: list[str | Path], metric: str, mode: str = "min") -> list[dict[str, Any]]:
    if mode not in ("min", "max"):
        raise ValueError("comparison mode must be min or max")
    missing = float("inf")

    def key(row: dict[str, Any]) -> float:
        value = row.get(metric)
        return float(value) if value is not None else missing
    return sorted((load_run_summary(d) for d in run_directories), key=key, reverse=(mode == "max"))


def write_comparison_csv(path: str | Path, results: list[dict[str, Any]]) -> Path:
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    columns = sorted({key for row in results for key in row})
    with target.open("w", encoding="utf-8", newline="") as handle:
        writer = csv.DictWriter(handle, fieldnames=columns)
        writer.writeheader()
        writer.writerows(results)
    return target
