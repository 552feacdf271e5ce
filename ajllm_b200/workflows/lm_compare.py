"""``lm compare``: rank an explicit list of finished runs (reference: ``ajllm/workflows/lm_compare.py:16-37``)."""

from __future__ import annotations

import json
from typing import Any

from ajllm_b200.artifacts import ArtifactPaths, write_manifest
from ajllm_b200.config import LoadedConfig
from ajllm_b200.evaluation import compare_runs, plot_learning_curves, write_comparison_csv
from ajllm_b200.workflows.common import project_path


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    name = str(data.get("name", "comparison"))
    runs = [project_path(config.project_root, p) for p in data.get("runs", [])]
    if not runs:
        raise ValueError("Comparison config requires at least one run directory")
    metric, mode = str(data.get("metric", "validation_loss")), str(data.get("mode", "min"))
    ranking = compare_runs(runs, metric, mode)
    out_dir = ArtifactPaths(config.project_root).task_run("comparisons", name)
    out_dir.mkdir(parents=True, exist_ok=True)
    write_comparison_csv(out_dir / "comparison.csv", ranking)
    if data.get("generate_plot", True):
        plot_learning_curves(runs, out_dir / "learning_curves.png")
    with (out_dir / "comparison.json").open("w", encoding="utf-8") as handle:
        json.dump(ranking, handle, indent=2, ensure_ascii=False)
    write_manifest(out_dir / "manifest.json", "run_comparison",
                   {"name": name, "metric": metric, "mode": mode, "run_count": len(ranking), "best_run": ranking[0]})
    return {"output_dir": str(out_dir), "results": ranking}
