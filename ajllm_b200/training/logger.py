"""Append-only JSON-lines metrics (reference: ``ajllm/training/logger.py:12-28``).

Each record is ``{step, event, wall_time_seconds, timestamp, **values}`` on one line of
``<run>/metrics.jsonl``; ``lm compare`` / ``lm sweep`` plots read these files.
"""

from __future__ import annotations

import json
import time
from datetime import datetime, timezone
from pathlib import Path
from typing import Any


class RunLogger:
    def __init__(self, run_directory: str | Path) -> None:
        self.run_directory = Path(run_directory)
        self.run_directory.mkdir(parents=True, exist_ok=True)
        self.metrics_path = self.run_directory / "metrics.jsonl"
        self._t0 = time.perf_counter()

    def log(self, step: int, event: str, values: dict[str, Any]) -> None:
        record: dict[str, Any] = {
            "step": int(step),
            "event": event,
            "wall_time_seconds": time.perf_counter() - self._t0,
            "timestamp": datetime.now(timezone.utc).isoformat(),
        }
        record.update(values)
        with self.metrics_path.open("a", encoding="utf-8") as handle:
            handle.write(json.dumps(record, ensure_ascii=False) + "\n")
