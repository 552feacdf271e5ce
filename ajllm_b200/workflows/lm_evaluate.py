"""``lm evaluate``: loss and perplexity of a saved run on an encoded split
(reference: ``ajllm/workflows/lm_evaluate.py:17-40``; writes ``runs/evaluations/<name>/<id>/result.json``)."""

from __future__ import annotations

from typing import Any

from ajllm_b200.artifacts import ArtifactPaths, open_encoded_artifact, write_manifest
from ajllm_b200.config import LoadedConfig
from ajllm_b200.evaluation import evaluate_model
from ajllm_b200.training import TokenDataset
from ajllm_b200.utils import pick_device
from ajllm_b200.workflows.common import load_model_from_run, project_path


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    name = str(data.get("name", "evaluation"))
    run_directory = project_path(config.project_root, data["run_directory"])
    device = pick_device(str(data.get("device", "auto")))
    model, train_cfg, _ = load_model_from_run(run_directory, str(data.get("checkpoint", "best")), device)
    enc_dir, enc_manifest = open_encoded_artifact(config.project_root, train_cfg["dataset"]["name"],
                                                  train_cfg["tokenizer"]["name"])
    split = str(data.get("split", "validation"))
    dataset = TokenDataset(enc_dir / enc_manifest["splits"][split]["path"])
    batch_size = int(data.get("batch_size", (train_cfg.get("training") or {}).get("batch_size", 32)))
    results = evaluate_model(model, dataset, int(data.get("batches", 100)), batch_size,
                             int(train_cfg["model"]["context_length"]), device, int(data.get("seed", 42)))
    out_dir = ArtifactPaths(config.project_root).task_run("evaluations", name)
    payload = {"training_run": str(run_directory), "split": split, **results}
    write_manifest(out_dir / "result.json", "evaluation", payload)
    return {"output_dir": str(out_dir), **payload}
