"""Where artifacts and runs live under a project root (reference: ``ajllm/artifacts/paths.py:11-39``).

Layout: ``artifacts/tokenizers/<name>``, ``artifacts/encoded/<dataset>/<tokenizer>``,
``runs/training/<dataset>/<tokenizer>/<model>/<experiment>/<run_id>``, ``runs/<task>/<name>/<run_id>``.
A run id is ``YYYYmmddTHHMMSSZ_<8 hex digits>``. In a multi-rank job rank 0 draws the id and
broadcasts it so that every rank writes into the same directory (the reference lets each rank draw
its own, ``ajllm/workflows/lm_train.py:43-50``).
"""

from __future__ import annotations

import secrets
from dataclasses import dataclass
from datetime import datetime, timezone
from pathlib import Path


def new_run_id() -> str:
    stamp = datetime.now(timezone.utc).strftime("%Y%m%dT%H%M%SZ")
    return f"{stamp}_{secrets.token_hex(4)}"


def shared_run_id() -> str:
    """Run id agreed on by all ranks of the default process group (rank 0 decides)."""
    import torch.distributed as dist

    run_id = new_run_id()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        box = [run_id]
        dist.broadcast_object_list(box, src=0)
        run_id = box[0]
    return run_id


@dataclass(frozen=True)
class ArtifactPaths:
    project_root: Path

    def tokenizer(self, name: str) -> Path:
        return self.project_root / "artifacts" / "tokenizers" / name

    def encoded(self, dataset: str, tokenizer: str) -> Path:
        return self.project_root / "artifacts" / "encoded" / dataset / tokenizer

    def training_run(self, dataset: str, tokenizer: str, model: str, experiment: str,
                     run_id: str | None = None) -> Path:
        leaf = run_id or shared_run_id()
        return self.project_root / "runs" / "training" / dataset / tokenizer / model / experiment / leaf

    def task_run(self, task: str, name: str, run_id: str | None = None) -> Path:
        return self.project_root / "runs" / task / name / (run_id or new_run_id())
