"""``lm sweep``: run ``lm train`` over the cartesian product of a grid of dotted-key overrides
(reference: ``ajllm/workflows/lm_sweep.py:17-88``; trial directories, ``comparison.csv``,
``trials.json``, learning curves and a manifest naming the best run)."""

from __future__ import annotations

import copy
import itertools
import json
from typing import Any

from ajllm_b200.artifacts import ArtifactPaths, write_manifest
from ajllm_b200.config import LoadedConfig, set_dotted_value
from ajllm_b200.evaluation import compare_runs, plot_learning_curves, write_comparison_csv
from ajllm_b200.workflows import lm_train


def trial_name(keys: list[str], values: tuple[Any, ...]) -> str:
    def clean(value: Any) -> str:
        return str(value).replace(".", "p").replace("+", "").replace("-", "m")
    return "__".join(f"{key.rsplit('.', 1)[-1]}_{clean(value)}" for key, value in zip(keys, values))


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    name = str(data.get("name", "sweep"))
    grid = data.get("grid")
    if not isinstance(grid, dict) or not grid:
        raise ValueError("Sweep config requires a non-empty grid mapping")
    keys = list(grid)
    axes = [v if isinstance(v, list) else [v] for v in grid.values()]
    out_dir = ArtifactPaths(config.project_root).task_run("sweeps", name)
    (out_dir / "trials").mkdir(parents=True, exist_ok=True)
    records, good_runs = [], []
    for values in itertools.product(*axes):
        label = trial_name(keys, values)
        overrides = dict(zip(keys, values))
        trial = copy.deepcopy(data)
        trial.pop("grid", None)
        trial.pop("name", None)
        trial["experiment"] = f"{name}_{label}"
        for key, value in overrides.items():
            set_dotted_value(trial, key, value)
        try:
            result = lm_train.run(config.replace_data(trial), out_dir / "trials" / label)
        except Exception as error:  # noqa: BLE001 - recorded per trial
            records.append({"name": label, "overrides": overrides, "status": "failed", "error": str(error)})
            if not data.get("continue_on_error", False):
                raise
            continue
        good_runs.append(result["run_directory"])
        records.append({"name": label, "overrides": overrides, **result})
    compare = data.get("comparison", {}) or {}
    metric, mode = str(compare.get("metric", "validation_loss")), str(compare.get("mode", "min"))
    ranking = compare_runs(good_runs, metric, mode) if good_runs else []
    write_comparison_csv(out_dir / "comparison.csv", ranking)
    if good_runs and compare.get("generate_plot", True):
        plot_learning_curves(good_runs, out_dir / "learning_curves.png")
    with (out_dir / "trials.json").open("w", encoding="utf-8") as handle:
        json.dump(records, handle, indent=2, ensure_ascii=False)
    best = ranking[0] if ranking else None
    write_manifest(out_dir / "manifest.json", "sweep",
                   {"name": name, "metric": metric, "mode": mode, "trial_count": len(records),
                    "successful_trial_count": len(good_runs), "best_run": best})
    return {"output_dir": str(out_dir), "trials": records, "best_run": best}
