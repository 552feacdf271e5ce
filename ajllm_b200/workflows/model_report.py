"""``model report``: write ``reports/models/<name>.md`` for a model component config
(reference: ``ajllm/workflows/model_report.py:12-31``; knobs ``report_vocab_size``, ``report_batch_size``,
``report_training_tokens``)."""

from __future__ import annotations

from typing import Any

from ajllm_b200.config import LoadedConfig
from ajllm_b200.models import build_model
from ajllm_b200.reporting import write_model_report


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    model_cfg = data.get("model", data)
    vocab_size = int(data.get("report_vocab_size", model_cfg.get("report_vocab_size", 10_000)))
    batch = int(data.get("report_batch_size", model_cfg.get("report_batch_size", 1)))
    training = dict(data.get("training", {}) or {})
    for source in (data, model_cfg):
        if "report_training_tokens" in source and "total_tokens" not in training:
            training["total_tokens"] = int(source["report_training_tokens"])
    training.setdefault("batch_size", batch)
    model = build_model(model_cfg, vocab_size)
    target = config.project_root / "reports" / "models" / f"{model_cfg['name']}.md"
    write_model_report(target, model, model_cfg, vocab_size, batch, training)
    return {"output_path": str(target), "model": model_cfg["name"], "vocab_size": vocab_size,
            "parameter_count": sum(p.numel() for p in model.parameters())}
