"""Learning curves from ``metrics.jsonl`` (reference: ``ajllm/evaluation/plotting.py:14-46``).

With matplotlib installed the figure is a PNG with training-loss and validation-loss panels (Agg
backend, headless). Without it, the same two panels are written as a standalone SVG next to the
requested path (same stem, ``.svg``), so sweeps and comparisons still produce a picture.
"""

from __future__ import annotations

import json
from pathlib import Path


def read_metrics(path: Path) -> list[dict]:
    with path.open("r", encoding="utf-8") as handle:
        return [json.loads(line) for line in handle if line.strip()]


def collect_curves(run_directories) -> list[dict]:
    curves = []
    for directory in run_directories:
        folder = Path(directory)
        records = read_metrics(folder / "metrics.jsonl")
        train = [(r["step"], r["loss"]) for r in records if r.get("event") == "train" and "loss" in r]
        val = [(r["step"], r["validation_loss"]) for r in records
               if r.get("event") == "evaluation" and "validation_loss" in r]
        curves.append({"label": f"{folder.parent.name}/{folder.name}", "train": train, "validation": val})
    return curves


def _svg_panel(x0: float, title: str, series: list[tuple[str, list[tuple[float, float]]]], width=560, height=360) -> str:
    pad = 48
    points = [p for _, pts in series for p in pts]
    parts = [f'<text x="{x0 + width / 2}" y="20" text-anchor="middle" font-size="14">{title}</text>',
             f'<rect x="{x0 + pad}" y="{pad}" width="{width - 2 * pad}" height="{height - 2 * pad}" fill="none" stroke="#888"/>']
    if points:
        xs, ys = [p[0] for p in points], [p[1] for p in points]
        x_lo, x_hi, y_lo, y_hi = min(xs), max(xs), min(ys), max(ys)
        x_span, y_span = (x_hi - x_lo) or 1.0, (y_hi - y_lo) or 1.0
        palette = ["#1f77b4", "#d62728", "#2ca02c", "#9467bd", "#ff7f0e", "#8c564b"]
        for index, (label, pts) in enumerate(series):
            if not pts:
                continue
            coords = " ".join(
                f"{x0 + pad + (x - x_lo) / x_span * (width - 2 * pad):.1f},"
                f"{height - pad - (y - y_lo) / y_span * (height - 2 * pad):.1f}" for x, y in pts)
            colour = palette[index % len(palette)]
            parts.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.5" points="{coords}"/>')
            parts.append(f'<text x="{x0 + pad + 6}" y="{pad + 14 + 12 * index}" font-size="9" fill="{colour}">{label}</text>')
        parts.append(f'<text x="{x0 + pad}" y="{height - pad + 14}" font-size="9">{x_lo:g}</text>')
        parts.append(f'<text x="{x0 + width - pad}" y="{height - pad + 14}" font-size="9" text-anchor="end">{x_hi:g}</text>')
        parts.append(f'<text x="{x0 + pad - 4}" y="{height - pad}" font-size="9" text-anchor="end">{y_lo:.3g}</text>')
        parts.append(f'<text x="{x0 + pad - 4}" y="{pad + 8}" font-size="9" text-anchor="end">{y_hi:.3g}</text>')
    return "\n".join(parts)


def plot_learning_curves(run_directories, output_path: str | Path) -> Path:
    curves = collect_curves(run_directories)
    target = Path(output_path)
    target.parent.mkdir(parents=True, exist_ok=True)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        target = target.with_suffix(".svg")
        body = _svg_panel(0, "Training Loss", [(c["label"], c["train"]) for c in curves]) + "\n" + \
            _svg_panel(580, "Validation Loss", [(c["label"], c["validation"]) for c in curves])
        target.write_text(f'<svg xmlns="http://www.w3.org/2000/svg" width="1160" height="360" '
                          f'font-family="sans-serif">\n{body}\n</svg>\n', encoding="utf-8")
        return target
    figure, axes = plt.subplots(1, 2, figsize=(13, 5))
    for curve in curves:
        if curve["train"]:
            axes[0].plot(*zip(*curve["train"]), label=curve["label"])
        if curve["validation"]:
            axes[1].plot(*zip(*curve["validation"]), marker="o", label=curve["label"])
    axes[0].set(title="Training Loss", xlabel="Step", ylabel="Cross-Entropy")
    axes[1].set(title="Validation Loss", xlabel="Step", ylabel="Cross-Entropy")
    for axis in axes:
        axis.grid(alpha=0.25)
        axis.legend(fontsize=7)
    figure.tight_layout()
    figure.savefig(target, dpi=180)
    plt.close(figure)
    return target
