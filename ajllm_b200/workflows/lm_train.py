"""``lm train``: build a self-contained training run (reference: ``ajllm/workflows/lm_train.py:25-199``).

Single process or one process per GPU under ``torchrun``. The ``parallel`` mapping chooses the mesh
(``tp`` x ``fsdp`` with ``ep`` inside the data-parallel axis); ``acceleration.use_fsdp: true`` without a
``parallel`` mapping means "shard over all ranks", as in the reference.

Precision. On the CPU the model trains in fp32, as the reference does by default. On a CUDA device every
configuration computes in bf16 on this package's kernels with fp32 master weights, fp32 gradients and fp32
optimizer state (any layout, not only FSDP): that is what ``acceleration.mixed_precision: bf16`` asks for,
what an absent key gets (the reference's fp32 default would leave the tensor cores idle and run none of the
kernels here), and what ``fp16`` is mapped to with a notice (same fp32 master weights, wider exponent, no
loss scaling needed). ``acceleration.fused`` (default true on CUDA) runs tensor-parallel projections and
the expert exchange as single kernels over symmetric NVLink memory instead of NCCL collectives.
All ranks share one run directory (rank 0 draws the id); rank 0 writes the report, manifest,
metrics and checkpoints.
"""

from __future__ import annotations

import os
from pathlib import Path
from typing import Any

import torch
import torch.distributed as dist

from ajllm_b200.artifacts import ArtifactPaths, open_encoded_artifact, open_tokenizer_artifact, write_manifest
from ajllm_b200.artifacts.registry import check_lineage
from ajllm_b200.config import LoadedConfig, check_dataset, check_model, check_parallel, check_tokenizer
from ajllm_b200.models import build_model
from ajllm_b200.reporting import write_model_report
from ajllm_b200.training import FlatAdamW, TokenDataset, Trainer
from ajllm_b200.utils import describe_device_choice, pick_device, seed_all
from ajllm_b200.workflows.common import dump_yaml


def _is_main() -> bool:
    return not dist.is_initialized() or dist.get_rank() == 0


def _optimizer_kwargs(data: dict[str, Any]) -> dict[str, Any]:
    opt = data.get("optimizer", {}) or {}
    return {"learning_rate": float(opt.get("max_lr", 1e-3)),
            "betas": (float(opt.get("beta1", 0.9)), float(opt.get("beta2", 0.95))),
            "epsilon": float(opt.get("epsilon", 1e-8)), "weight_decay": float(opt.get("weight_decay", 0.1))}


def run(config: LoadedConfig, run_directory: Path | None = None) -> dict[str, Any]:
    data = config.data
    dataset_cfg, tokenizer_cfg, model_cfg = data["dataset"], data["tokenizer"], data["model"]
    check_dataset(dataset_cfg)
    check_tokenizer(tokenizer_cfg)
    check_model(model_cfg)
    tok_dir, tok_manifest = open_tokenizer_artifact(config.project_root, tokenizer_cfg["name"])
    enc_dir, enc_manifest = open_encoded_artifact(config.project_root, dataset_cfg["name"], tokenizer_cfg["name"])
    check_lineage(tok_manifest, enc_manifest)

    runtime = data.get("runtime", {}) or {}
    seed = int(runtime.get("seed", 42))
    requested = str(runtime.get("device", "auto"))
    device = pick_device(requested)
    acceleration = data.get("acceleration", {}) or {}
    use_fsdp = bool(acceleration.get("use_fsdp", False))
    mixed = acceleration.get("mixed_precision")
    parallel_cfg = data.get("parallel", {}) or {}
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if use_fsdp and "RANK" not in os.environ:
        raise RuntimeError("FSDP requires a distributed environment. Launch with torchrun or lm_train_distributed")
    if world > 1:
        from ajllm_b200.parallel import init_distributed
        _, _, device = init_distributed(device.type)
    precision_note = None
    if mixed is not None:
        if mixed not in ("fp16", "bf16"):
            raise ValueError(f"mixed_precision must be 'fp16', 'bf16', or null, got: {mixed}")
        if device.type != "cuda":
            raise ValueError(f"Mixed precision requires a CUDA device, got: {device.type}")
        if mixed == "fp16":
            precision_note = "fp16 was requested: computing in bf16 with fp32 master weights (no loss scaling needed)"
    elif device.type == "cuda":
        precision_note = "no mixed_precision key: a CUDA device computes in bf16 with fp32 master weights and optimizer state"
    compute_dtype = torch.bfloat16 if device.type == "cuda" else torch.float32
    seed_all(seed)

    experiment = str(data.get("experiment", "training"))
    run_directory = run_directory or ArtifactPaths(config.project_root).training_run(
        dataset_cfg["name"], tokenizer_cfg["name"], model_cfg["name"], experiment, data.get("run_id"))
    vocab_size = int(tok_manifest["vocab_size"])
    data["_runtime"] = {"vocab_size": vocab_size, "tokenizer_directory": str(tok_dir),
                        "encoded_directory": str(enc_dir), "run_directory": str(run_directory)}
    resume_from = (data.get("training", {}) or {}).get("resume_from")
    if resume_from:
        resume_path = Path(str(resume_from))
        if not resume_path.is_absolute():
            resume_path = (config.project_root / resume_path).resolve()
        data["training"]["resume_from"] = str(resume_path)
    if _is_main():
        run_directory.mkdir(parents=True, exist_ok=True)
        dump_yaml(run_directory / "resolved_config.yaml", data)
    if world > 1:
        dist.barrier()

    splits = data.get("data_splits", {"train": "train", "validation": "validation"})
    train_dataset = TokenDataset(enc_dir / enc_manifest["splits"][splits["train"]]["path"])
    val_name = splits.get("validation")
    validation_dataset = (TokenDataset(enc_dir / enc_manifest["splits"][val_name]["path"])
                          if val_name and val_name in enc_manifest["splits"] else None)

    # ---- mesh and model
    tp = ep = cp = None
    mesh = None
    sizes = {"tp": 1, "ep": 1, "fsdp": 1, "pp": 1, "cp": 1}
    if world > 1:
        from ajllm_b200.parallel import ParallelMesh
        from ajllm_b200.parallel.contexts import make_expert_parallel, make_tensor_parallel
        defaults = dict(parallel_cfg)
        if "fsdp" not in defaults and "tp" not in defaults and "cp" not in defaults:
            defaults["fsdp"] = world
        sizes = check_parallel(defaults, world)
        if sizes["pp"] != 1 and (sizes["tp"] != 1 or sizes["fsdp"] != 1 or sizes["ep"] != 1):
            raise ValueError("pipeline parallelism runs on its own here: set tp = fsdp = ep = 1 (pp = world size)")
        # context-parallel peers take the innermost (adjacent-rank) axis, the one tensor parallelism would use
        mesh = ParallelMesh(tp=sizes["tp"] * sizes["cp"], fsdp=sizes["fsdp"], ep=sizes["ep"], pp=sizes["pp"])
        if sizes["cp"] > 1:
            if use_fsdp:
                raise ValueError("context parallelism runs with replicated data parallelism (acceleration.use_fsdp: false)")
            from ajllm_b200.parallel.context_parallel import ContextParallel
            cp = ContextParallel(mesh.tp.group, mesh.tp.rank, mesh.tp.size)
        fused = acceleration.get("fused")
        if cp is None:
            tp = make_tensor_parallel(mesh.tp, device, None if fused is None else bool(fused))
        ep = make_expert_parallel(mesh.ep, device, None if fused is None else bool(fused))
    from ajllm_b200.parallel.contexts import expert_exchange_backend, tp_backend
    checkpointing = str(acceleration.get("activation_checkpointing", "layer" if use_fsdp else "none"))
    dtype = compute_dtype
    model = build_model(model_cfg, vocab_size, bool(acceleration.get("use_flash_attention", False)), tp=tp, ep=ep, cp=cp,
                        activation_checkpointing="none" if use_fsdp else checkpointing)
    model = model.to(device=device, dtype=dtype)
    parameter_count = sum(p.numel() for p in model.parameters())
    base_model = model
    # the report describes the whole model: written before any wrapper shards or splits the parameters, from gathered
    # tensors (a collective, hence on every rank) when tensor or expert parallelism holds only a part of them here
    whole_state = base_model.state_dict() if (tp is not None or ep is not None) else None
    if _is_main():
        training_for_report = data.get("training", {}) or {}
        write_model_report(run_directory / "model_report.md", base_model, model_cfg, vocab_size,
                           int(training_for_report.get("batch_size", 64)), training_for_report, state_dict=whole_state)
    del whole_state

    optimizer = None
    dp_size = mesh.dp_size if mesh is not None else 1
    dp_rank = mesh.dp_index if mesh is not None else 0
    loss_group = None
    if mesh is not None and sizes["pp"] > 1:
        from ajllm_b200.parallel import PipelineOptimizer, PipelineParallel
        micro = int((data.get("parallel", {}) or {}).get("pp_microbatches", sizes["pp"]))
        model = PipelineParallel(model, mesh.pp.group, micro)
        optimizer = PipelineOptimizer(model, **_optimizer_kwargs(data))
    elif mesh is not None and use_fsdp and dp_size > 1:
        from ajllm_b200.parallel.fsdp import ShardedDataParallel
        model = ShardedDataParallel(model, mesh.dp.group, checkpoint_layers=(checkpointing != "none"),
                                    **_optimizer_kwargs(data))
        optimizer = model.optimizer
        loss_group = mesh.dp.group
    elif mesh is not None:
        from ajllm_b200.parallel.data_parallel import optimizer_classes
        optimizer = FlatAdamW(model, classes=optimizer_classes(mesh, tp, cp), **_optimizer_kwargs(data))
        loss_group = mesh.dp.group if dp_size > 1 else None
        if dp_size > 1:
            model.data_parallel_share = 1.0 / dp_size

    training_cfg = data.get("training", {}) or {}
    batch_size = int(training_cfg.get("batch_size", 64))
    context_length = int(base_model.context_length)
    if _is_main():
        print("Training setup:")
        print(f"  device: {device} (requested: {requested})")
        note = describe_device_choice(requested, device)
        if note:
            print(f"  device note: {note}")
        print(f"  world size: {world}  mesh: tp={sizes['tp']} cp={sizes['cp']} fsdp={sizes['fsdp']} ep={sizes['ep']}")
        print(f"  train tokens: {len(train_dataset):,}")
        if validation_dataset is not None:
            print(f"  validation tokens: {len(validation_dataset):,}")
        print(f"  batch size per data-parallel rank: {batch_size:,}  context length: {context_length:,}")
        print(f"  gradient accumulation: {int(training_cfg.get('gradient_accumulation_steps', 1))}")
        print(f"  model parameters on this rank: {parameter_count:,}")
        print(f"  FSDP: {'enabled' if use_fsdp else 'disabled'}  mixed precision: {mixed or 'disabled'}")
        print(f"  compute dtype: {str(dtype).replace('torch.', '')}  master weights / optimizer state: float32")
        if precision_note:
            print(f"  precision note: {precision_note}")
        print(f"  tensor-parallel projections: {tp_backend(tp)}  expert exchange: {expert_exchange_backend(ep)}")
        print(f"  activation checkpointing: {checkpointing}")
    manifest = {"experiment": experiment, "dataset": dataset_cfg["name"], "tokenizer": tokenizer_cfg["name"],
                "model": model_cfg["name"], "parameter_count": parameter_count, "device": str(device),
                "world_size": world, "parallel": sizes, "compute_dtype": str(dtype).replace("torch.", ""),
                "tp_backend": tp_backend(tp), "expert_exchange": expert_exchange_backend(ep)}
    if _is_main():
        write_manifest(run_directory / "manifest.json", "training_run", manifest)
    trainer = Trainer(model, train_dataset, validation_dataset, run_directory, data, device, seed, optimizer=optimizer,
                      data_rank=dp_rank, data_world=dp_size, loss_reduce_group=loss_group)
    summary = trainer.train({**manifest, "resolved_config": data, "vocab_size": vocab_size})
    return {"run_directory": str(run_directory), **manifest, **summary}
