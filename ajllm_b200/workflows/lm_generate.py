"""``lm generate``: sample completions from a saved run (reference:
``ajllm/workflows/lm_generate.py:23-104``; same config keys and ``results.json`` / ``manifest.json``).

All prompts and their ``samples_per_prompt`` copies are submitted to the continuous-batching engine at
once instead of being generated one after another; ``engine:`` may set ``block_size``,
``max_num_seqs``, ``quantization: fp8`` and ``speculative: {draft_run_directory, k}``.

Launched with one process per GPU (``torchrun``), the model is served tensor-parallel over all ranks:
every rank loads its slice of the checkpoint, row-parallel projections end in the fused
GEMM -> all-reduce kernel (``acceleration.fused: false`` or ``AJB_FUSED_TP=0``: NCCL), every rank runs
the same scheduler and sampler from the same seeds, and rank 0 writes the results.
"""

from __future__ import annotations

import json
import os
import time
from pathlib import Path
from typing import Any

from ajllm_b200.artifacts import ArtifactPaths, open_tokenizer_artifact, write_manifest
from ajllm_b200.config import LoadedConfig
from ajllm_b200.engine import LLMEngine, SamplingParams
from ajllm_b200.tokenization import Tokenizer
from ajllm_b200.utils import pick_device, seed_all
from ajllm_b200.workflows.common import load_model_from_run, project_path


def read_prompts(data: dict[str, Any], project_root: Path) -> list[str]:
    if "prompts" in data:
        return [str(p) for p in data["prompts"]]
    if "prompt_file" in data:
        text = project_path(project_root, data["prompt_file"]).read_text(encoding="utf-8")
        return [line.strip() for line in text.splitlines() if line.strip()]
    raise ValueError("Generation config requires prompts or prompt_file")


def run(config: LoadedConfig) -> dict[str, Any]:
    data = config.data
    name = str(data.get("name", "generation"))
    training_run = project_path(config.project_root, data["run_directory"])
    device = pick_device(str(data.get("device", "auto")))
    seed = int(data.get("seed", 42))
    seed_all(seed)
    checkpoint = str(data.get("checkpoint", "best"))
    tp = None
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1:
        from ajllm_b200.parallel import ParallelMesh, init_distributed
        from ajllm_b200.parallel.contexts import make_tensor_parallel
        _, _, device = init_distributed(device.type)
        fused = (data.get("acceleration", {}) or {}).get("fused")
        tp = make_tensor_parallel(ParallelMesh(tp=world).tp, device, None if fused is None else bool(fused), interleave=1)
    main = tp is None or tp.rank == 0
    model, train_cfg, _ = load_model_from_run(training_run, checkpoint, device, tp=tp)
    tok_dir, tok_manifest = open_tokenizer_artifact(config.project_root, train_cfg["tokenizer"]["name"])
    tokenizer = Tokenizer.from_files(tok_dir / tok_manifest["files"]["vocab"], tok_dir / tok_manifest["files"]["merges"],
                                     tok_manifest.get("special_tokens", []))
    max_new = int(data.get("max_new_tokens", 100))
    temperature = float(data.get("temperature", 0.8))
    top_p = data.get("top_p", 0.95)
    top_p = None if top_p is None else float(top_p)
    samples = int(data.get("samples_per_prompt", 1))
    eos_id = tokenizer.token_to_id.get(str(data.get("eos_token", "<|endoftext|>")).encode("utf-8"))

    engine_cfg = data.get("engine", {}) or {}
    draft, k = None, 0
    spec = engine_cfg.get("speculative") or {}
    if spec.get("draft_run_directory"):
        draft, _, _ = load_model_from_run(project_path(config.project_root, spec["draft_run_directory"]),
                                          str(spec.get("checkpoint", "best")), device, tp=tp)
        k = int(spec.get("k", 4))
    engine = LLMEngine(model, block_size=int(engine_cfg.get("block_size", 16)),
                       max_num_seqs=int(engine_cfg.get("max_num_seqs", 256)),
                       quantization=engine_cfg.get("quantization"), draft_model=draft,
                       num_speculative_tokens=k or 4, seed=seed)
    prompts = read_prompts(data, config.project_root)
    encoded = [tokenizer.encode(p) or ([eos_id] if eos_id is not None else [0]) for p in prompts]
    requests, owners = [], []
    for index, ids in enumerate(encoded):
        room = max(1, min(max_new, model.context_length + 1 - len(ids)))
        for sample in range(samples):
            requests.append((ids, SamplingParams(room, temperature, top_p, eos_id,
                                                 seed=seed * 1_000_003 + index * 1009 + sample)))
            owners.append(index)
    started = time.perf_counter()
    outputs = engine.generate([r[0] for r in requests], [r[1] for r in requests])
    elapsed = time.perf_counter() - started
    results = [{"prompt": p, "completions": []} for p in prompts]
    for owner, (ids, _), out in zip(owners, requests, outputs):
        full = list(out.prompt) + list(out.output)
        results[owner]["completions"].append({
            "text": tokenizer.decode(full), "token_count": len(full),
            "elapsed_seconds": out.latency_seconds if out.latency_seconds is not None else elapsed,
        })
    from ajllm_b200.parallel.contexts import tp_backend
    out_dir = ArtifactPaths(config.project_root).task_run("generations", name)
    payload = {
        "training_run": str(training_run), "checkpoint": checkpoint,
        "parameters": {"max_new_tokens": max_new, "temperature": temperature, "top_p": top_p,
                       "samples_per_prompt": samples, "seed": seed},
        "throughput": {"output_tokens": engine.stats.output_tokens, "elapsed_seconds": elapsed,
                       "output_tokens_per_second": engine.stats.output_tokens / max(elapsed, 1e-9)},
        "tensor_parallel": {"size": world, "backend": tp_backend(tp)},
        "results": results,
    }
    if main:
        out_dir.mkdir(parents=True, exist_ok=True)
        with (out_dir / "results.json").open("w", encoding="utf-8") as handle:
            json.dump(payload, handle, indent=2, ensure_ascii=False)
        write_manifest(out_dir / "manifest.json", "generation", {k_: v for k_, v in payload.items() if k_ != "results"})
    return {"output_dir": str(out_dir), **payload}
