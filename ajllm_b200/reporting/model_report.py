"""Markdown report of a model: diagram, dimensions, shapes, parameters, memory and FLOPs.

Section titles and table rows follow the reference report (``ajllm/reporting/model_report.py:57-174``)
so existing readers of ``model_report.md`` keep working; the parameter table lists the checkpoint key
names (the fused q|k|v and gate|up storage is an implementation detail), grouped KV heads and MoE
layers are described, and a B200 time estimate is appended.
"""

from __future__ import annotations

from pathlib import Path
from typing import Any

import torch

from ajllm_b200.reporting.resource_estimates import ResourceEstimate, estimate_resources

# measured on the target machines (cuBLAS bf16 sustained, STREAM-like copy)
B200_BF16_FLOPS = 1.39e15
B200_HBM_BYTES_PER_S = 6.54e12


def parameter_formula(model_config: dict[str, Any]) -> str:
    ff = (model_config.get("feed_forward") or {}).get("type", "swiglu")
    norm = model_config.get("normalization") or {}
    heads = int(model_config["num_heads"])
    kv = int(model_config.get("num_kv_heads", heads))
    attention = "4D^2" if kv == heads else "2D^2 + 2D·(Hkv·D/H)"
    if model_config.get("moe"):
        ffn = "E·3DF + S·3DF + ED"
    else:
        ffn = f"{3 if ff == 'swiglu' else 2}DF"
    per_layer = f"{attention} + {ffn}" + (" + 2D" if norm.get("type", "rmsnorm") == "rmsnorm" else "")
    head = "VD" if model_config.get("tie_embeddings", False) else "2VD"
    positions = " + TD" if (model_config.get("position_encoding") or {}).get("type") == "learned" else ""
    final = " + D" if norm.get("type", "rmsnorm") == "rmsnorm" and norm.get("placement", "pre") == "pre" else ""
    return f"N = {head}{positions} + L({per_layer}){final}"


def human_bytes(value: int) -> str:
    gib = value / 2**30
    return f"{value:,} bytes ({gib:.3f} GiB)" if gib >= 1 else f"{value:,} bytes ({value / 2**20:.3f} MiB)"


def human_flops(value: int) -> str:
    for scale, unit in ((1e15, "PFLOPs"), (1e12, "TFLOPs"), (1e9, "GFLOPs")):
        if value >= scale:
            return f"{value / scale:.3f} {unit}"
    return f"{value:,} FLOPs"


def _table(header: tuple[str, ...], align: str, rows: list[tuple]) -> str:
    lines = ["| " + " | ".join(header) + " |", align]
    lines += ["| " + " | ".join(str(cell) for cell in row) + " |" for row in rows]
    return "\n".join(lines)


def _memory_table(r: ResourceEstimate) -> str:
    return _table(("Component", "Estimate"), "|---|---:|", [
        ("Parameters", human_bytes(r.parameter_bytes)),
        ("Saved activations (estimated)", human_bytes(r.activation_bytes)),
        ("Parameter gradients", human_bytes(r.gradient_bytes)),
        ("AdamW first and second moments", human_bytes(r.optimizer_bytes)),
        ("Total estimated training memory", human_bytes(r.total_memory_bytes)),
    ])


def write_model_report(path: str | Path, model: torch.nn.Module, model_config: dict[str, Any], vocab_size: int,
                       batch_size: int | str = "B", training_config: dict[str, Any] | None = None,
                       state_dict: dict[str, torch.Tensor] | None = None) -> Path:
    """``state_dict``: the whole model's tensors when ``model`` holds only this rank's part of them (under tensor or
    expert parallelism gathering them is a collective, so the caller does it on every rank and passes the result)."""
    target = Path(path)
    target.parent.mkdir(parents=True, exist_ok=True)
    T, D = int(model_config["context_length"]), int(model_config["d_model"])
    H, L = int(model_config["num_heads"]), int(model_config["num_layers"])
    Hkv = int(model_config.get("num_kv_heads", H))
    F, hd = int(getattr(model, "d_ff")), D // H
    named = list((state_dict if state_dict is not None else model.state_dict()).items())
    total = sum(t.numel() for _, t in named) if state_dict is not None else sum(p.numel() for p in model.parameters())
    numeric_batch = int(batch_size) if isinstance(batch_size, int) else int(model_config.get("report_batch_size", 1))
    shown_batch = batch_size if isinstance(batch_size, int) else f"{batch_size} (estimate uses {numeric_batch})"
    flash = next(model.parameters()).is_cuda
    r = estimate_resources({**model_config, "vocab_size": vocab_size}, total, numeric_batch, training_config,
                           flash_attention=flash)
    moe = model_config.get("moe")
    ffn_text = (f"a mixture of {moe['num_experts']} experts (top-{moe['top_k']}, {moe.get('shared_experts', 0)} shared)"
                if moe else "a feed-forward network")

    sections = [f"# Model Architecture: {model_config.get('name', 'transformer')}",
                "This report is generated from the resolved model configuration and instantiated model.",
                "\n".join(["```mermaid", "flowchart LR",
                           '    A["Token IDs [B, T]"] --> B["Token Embedding [B, T, D]"]',
                           f'    B --> C["Transformer Blocks x {L}"]',
                           '    C --> D["Final Normalization [B, T, D]"]',
                           '    D --> E["LM Head [B, T, V]"]', "```"]),
                f"Each Transformer block contains causal self-attention ({H} query heads, {Hkv} key/value heads) and "
                f"{ffn_text} connected by residual paths. Normalization placement and position encoding are "
                "controlled by the model configuration.",
                "## Configured Dimensions",
                _table(("Symbol", "Meaning", "Value"), "|---|---|---:|", [
                    ("B", "Batch size", shown_batch), ("T", "Context length", T), ("V", "Vocabulary size", vocab_size),
                    ("D", "Model width", D), ("L", "Transformer layers", L), ("H", "Attention heads", H),
                    ("Hkv", "Key/value heads", Hkv), ("D/H", "Head dimension", hd), ("F", "Feed-forward width", F)]),
                "## Tensor Shapes",
                _table(("Stage", "Shape"), "|---|---|", [
                    ("Input token IDs", f"`[{shown_batch}, {T}]`"),
                    ("Token embeddings", f"`[{shown_batch}, {T}, {D}]`"),
                    ("Q per head", f"`[{shown_batch}, {H}, {T}, {hd}]`"),
                    ("K, V per head", f"`[{shown_batch}, {Hkv}, {T}, {hd}]`"),
                    ("Attention scores", f"`[{shown_batch}, {H}, {T}, {T}]`" + (" (never stored: tiled kernel)" if flash else "")),
                    ("Block output", f"`[{shown_batch}, {T}, {D}]`"),
                    ("LM logits", f"`[{shown_batch}, {T}, {vocab_size}]`")]),
                "## Parameters",
                "General formula for the selected architecture:",
                f"```text\n{parameter_formula(model_config)}\n```",
                f"Instantiated parameter count: **{total:,}**.",
                _table(("Parameter", "Shape", "Count"), "|---|---|---:|",
                       [(f"`{name}`", f"`{list(t.shape)}`", f"{t.numel():,}") for name, t in named]),
                "## Estimated Training Memory",
                _memory_table(r),
                f"The estimate uses parameter/gradient dtype size `{r.parameter_dtype_bytes}` bytes, activation dtype size "
                f"`{r.activation_dtype_bytes}` bytes, and `{r.optimizer_state_dtype_bytes}` bytes per AdamW moment. It "
                "excludes CUDA workspaces, allocator fragmentation, data-loader memory, and framework overhead.",
                "## Estimated Matrix FLOPs",
                _table(("Quantity", "Estimate"), "|---|---:|", [
                    ("Forward FLOPs per iteration", human_flops(r.forward_flops_per_step)),
                    ("Training FLOPs per iteration (3x forward approximation)", human_flops(r.training_flops_per_step)),
                    ("Planned training steps", r.total_training_steps or "not specified"),
                    ("Planned training tokens", r.total_training_tokens or "not specified"),
                    ("Total training FLOPs", human_flops(r.total_training_flops) if r.total_training_flops else "not specified"),
                    ("Iteration time at the measured B200 bf16 GEMM rate (lower bound, one GPU)",
                     f"{r.training_flops_per_step / B200_BF16_FLOPS * 1e3:.3f} ms")]),
                "The FLOPs estimate counts matrix multiplications only: Q/K/V/output projections, attention QK^T and AV "
                "products, feed-forward projections, and the LM head. Elementwise activation, normalization, masking, "
                "sampling, and optimizer arithmetic are omitted."]
    target.write_text("\n\n".join(sections) + "\n", encoding="utf-8")
    return target
