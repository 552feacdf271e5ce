"""Benchmark of the acceleration options: phase times, peak memory and throughput per configuration.

Counterpart of the reference's ``ajllm/workflows/benchmark_distributed.py`` (four configurations x the phases
forward / backward / optimizer / total, JSON + CSV + figure). The configurations keep the reference's names; here
they select:

* ``baseline``                  fp32 parameters, plain PyTorch math requested explicitly (``ops.eager_cuda()``; without
                                that request an fp32 CUDA tensor is refused by the ops layer),
* ``flash_attention``           bf16 parameters: the tcgen05 GEMM / attention / fused pointwise kernels,
* ``fsdp_ac``                   ``baseline`` under fully sharded data parallelism with per-layer recomputation,
* ``flash_attention_fsdp_ac``   ``flash_attention`` under the same wrapper.

Phases are timed on the device (CUDA events on the current stream, a synchronize on both sides) or with the host
clock on CPUs. The sharded wrapper runs forward and backward inside one call, so for the two sharded
configurations "forward" is a separate evaluation-mode pass and "backward" is the training call minus that pass.

    python -m ajllm_b200.workflows.benchmark_distributed --device cuda --steps 5 --warmup 2
    python -m ajllm_b200.workflows.benchmark_distributed --device cuda --world-size 2 --configs fsdp_ac flash_attention_fsdp_ac
    python -m ajllm_b200.workflows.benchmark_distributed --device cpu --d-model 64 --num-layers 2 --num-heads 4 --batch-size 4 --context-length 32
"""

from __future__ import annotations

import argparse
import csv
import json
import os
import statistics
import time
from dataclasses import asdict, dataclass
from pathlib import Path

import torch
import torch.distributed as dist

CONFIGS = ("baseline", "flash_attention", "fsdp_ac", "flash_attention_fsdp_ac")
PHASES = ("forward", "backward", "optimizer", "total")


@dataclass
class PhaseStats:
    mean_ms: float
    std_ms: float
    peak_memory_mb: float


@dataclass
class BenchmarkResult:
    config: str
    device: str
    world_size: int
    rank: int
    vocab_size: int
    d_model: int
    num_layers: int
    num_heads: int
    batch_size: int
    context_length: int
    steps: int
    warmup_steps: int
    forward: PhaseStats
    backward: PhaseStats
    optimizer: PhaseStats
    total: PhaseStats
    parameter_count: int
    tokens_per_second: float


def parse_args(argv=None) -> argparse.Namespace:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--device", choices=("cpu", "cuda"), default="cuda")
    ap.add_argument("--configs", nargs="+", choices=CONFIGS, default=list(CONFIGS))
    ap.add_argument("--world-size", type=int, default=1, help="ranks for the sharded configurations")
    ap.add_argument("--vocab-size", type=int, default=10000)
    ap.add_argument("--d-model", type=int, default=512)
    ap.add_argument("--num-layers", type=int, default=4)
    ap.add_argument("--num-heads", type=int, default=16)
    ap.add_argument("--batch-size", type=int, default=32)
    ap.add_argument("--context-length", type=int, default=256)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=2)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--master-port", type=str, default="29501")
    ap.add_argument("--output-dir", type=Path, default=Path("results"))
    return ap.parse_args(argv)


class _Clock:
    """Elapsed milliseconds between ``start`` and ``stop``: CUDA events on a GPU, the host clock otherwise."""

    def __init__(self, device: torch.device) -> None:
        self.device = device
        self.cuda = device.type == "cuda"

    def start(self) -> None:
        if self.cuda:
            torch.cuda.synchronize(self.device)
            torch.cuda.reset_peak_memory_stats(self.device)
            self._begin = torch.cuda.Event(enable_timing=True)
            self._begin.record()
        else:
            self._t0 = time.perf_counter()

    def stop(self) -> tuple[float, float]:
        if self.cuda:
            end = torch.cuda.Event(enable_timing=True)
            end.record()
            torch.cuda.synchronize(self.device)
            return self._begin.elapsed_time(end), torch.cuda.max_memory_allocated(self.device) / 2 ** 20
        return (time.perf_counter() - self._t0) * 1e3, 0.0


def _stats(samples: list[float], peaks: list[float]) -> PhaseStats:
    return PhaseStats(statistics.mean(samples), statistics.stdev(samples) if len(samples) > 1 else 0.0,
                      max(peaks) if peaks else 0.0)


def _worker(args: argparse.Namespace, config: str, rank: int, world: int) -> BenchmarkResult:
    import contextlib

    from ajllm_b200.ops.functional import eager_cuda

    # the two fp32 arms are the eager-PyTorch baselines of the comparison
    with (contextlib.nullcontext() if "flash_attention" in config else eager_cuda()):
        return _worker_body(args, config, rank, world)


def _worker_body(args: argparse.Namespace, config: str, rank: int, world: int) -> BenchmarkResult:
    from ajllm_b200.models import build_model
    from ajllm_b200.training.optim import FlatAdamW

    use_cuda = args.device == "cuda"
    if use_cuda and not torch.cuda.is_available():
        raise RuntimeError("CUDA requested but not available")
    device = torch.device("cuda", rank % torch.cuda.device_count()) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ["MASTER_PORT"] = args.master_port
        kwargs = {"device_id": device} if use_cuda else {}
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world, **kwargs)
    try:
        native = "flash_attention" in config
        sharded = "fsdp" in config
        dtype = torch.bfloat16 if (native and use_cuda) else torch.float32
        model_cfg = {"name": "bench", "context_length": args.context_length, "d_model": args.d_model,
                     "num_layers": args.num_layers, "num_heads": args.num_heads, "d_ff": 4 * args.d_model}
        torch.manual_seed(42)
        model = build_model(model_cfg, args.vocab_size, native).to(device=device, dtype=dtype)
        parameter_count = sum(p.numel() for p in model.parameters())
        if sharded and world > 1:
            from ajllm_b200.parallel.fsdp import ShardedDataParallel
            model = ShardedDataParallel(model, dist.group.WORLD, checkpoint_layers=True, learning_rate=args.lr)
            optimizer = model.optimizer
        else:
            optimizer = FlatAdamW(model, args.lr, (0.9, 0.95), 1e-8, 0.0)
        torch.manual_seed(1234)
        local_batch = max(1, args.batch_size // (world if sharded else 1))
        tokens = torch.randint(0, args.vocab_size, (local_batch, args.context_length + 1), device=device)
        inputs, targets = tokens[:, :-1], tokens[:, 1:]
        wrapped = sharded and world > 1
        clock = _Clock(device)
        times = {p: [] for p in PHASES}
        peaks = {p: [] for p in PHASES}
        for step in range(args.warmup + args.steps):
            optimizer.zero_grad()
            if wrapped:
                clock.start()
                with torch.no_grad():
                    model.loss(inputs, targets)
                fwd_ms, fwd_peak = clock.stop()
                clock.start()
                model.loss(inputs, targets)
                both_ms, bwd_peak = clock.stop()
                bwd_ms = max(0.0, both_ms - fwd_ms)
            else:
                clock.start()
                loss = model.loss(inputs, targets)
                fwd_ms, fwd_peak = clock.stop()
                clock.start()
                loss.backward()
                bwd_ms, bwd_peak = clock.stop()
            clock.start()
            optimizer.step(1.0)
            opt_ms, opt_peak = clock.stop()
            if step >= args.warmup:
                for phase, ms, peak in (("forward", fwd_ms, fwd_peak), ("backward", bwd_ms, bwd_peak),
                                        ("optimizer", opt_ms, opt_peak),
                                        ("total", fwd_ms + bwd_ms + opt_ms, max(fwd_peak, bwd_peak, opt_peak))):
                    times[phase].append(ms)
                    peaks[phase].append(peak)
        total = _stats(times["total"], peaks["total"])
        tokens_per_step = local_batch * args.context_length * (world if sharded else 1)
        return BenchmarkResult(config, str(device), world if sharded else 1, rank, args.vocab_size, args.d_model, args.num_layers,
                               args.num_heads, args.batch_size, args.context_length, args.steps, args.warmup,
                               _stats(times["forward"], peaks["forward"]), _stats(times["backward"], peaks["backward"]),
                               _stats(times["optimizer"], peaks["optimizer"]), total, parameter_count,
                               tokens_per_step / (total.mean_ms / 1e3))
    finally:
        if world > 1 and dist.is_initialized():
            dist.barrier()
            dist.destroy_process_group()


def _spawned(rank: int, args: argparse.Namespace, config: str, queue) -> None:
    queue.put(asdict(_worker(args, config, rank, args.world_size)))


def _restore(data: dict) -> BenchmarkResult:
    for phase in PHASES:
        data[phase] = PhaseStats(**data[phase])
    return BenchmarkResult(**data)


def run_config(args: argparse.Namespace, config: str) -> list[BenchmarkResult]:
    world = args.world_size if "fsdp" in config else 1
    if world == 1:
        return [_worker(args, config, 0, 1)]
    import torch.multiprocessing as mp
    queue = mp.get_context("spawn").SimpleQueue()
    mp.spawn(_spawned, args=(args, config, queue), nprocs=world, join=True)
    return sorted((_restore(queue.get()) for _ in range(world)), key=lambda r: r.rank)


def _bars_svg(path: Path, title: str, labels: list[str], series: dict[str, list[float]], unit: str) -> None:
    """Grouped bars without any plotting library."""
    width, height, left, bottom = 720, 360, 70, 60
    top = max((v for vals in series.values() for v in vals), default=1.0) or 1.0
    colours = ["#4c72b0", "#dd8452", "#55a868", "#c44e52"]
    parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{width}" height="{height}" font-family="sans-serif" font-size="11">',
             f'<text x="{width / 2}" y="18" text-anchor="middle" font-size="14">{title}</text>']
    group = (width - left - 20) / max(1, len(labels))
    bar = group / (len(series) + 1)
    for gi, label in enumerate(labels):
        parts.append(f'<text x="{left + gi * group + group / 2}" y="{height - bottom + 16}" text-anchor="middle">{label}</text>')
        for si, (name, values) in enumerate(series.items()):
            h = (height - bottom - 40) * values[gi] / top
            x = left + gi * group + si * bar + bar / 2
            parts.append(f'<rect x="{x:.1f}" y="{height - bottom - h:.1f}" width="{bar * 0.9:.1f}" height="{h:.1f}" fill="{colours[si % 4]}"/>')
    for si, name in enumerate(series):
        parts.append(f'<rect x="{left + si * 150}" y="{height - 22}" width="10" height="10" fill="{colours[si % 4]}"/>'
                     f'<text x="{left + si * 150 + 14}" y="{height - 13}">{name}</text>')
    parts.append(f'<text x="12" y="{height / 2}" transform="rotate(-90 12 {height / 2})" text-anchor="middle">{unit}</text></svg>')
    path.write_text("\n".join(parts), encoding="utf-8")


def write_outputs(args: argparse.Namespace, results: list[BenchmarkResult]) -> dict[str, str]:
    out = Path(args.output_dir)
    out.mkdir(parents=True, exist_ok=True)
    json_path = out / "benchmark_acceleration.json"
    json_path.write_text(json.dumps([asdict(r) for r in results], indent=2) + "\n", encoding="utf-8")
    csv_path = out / "benchmark_acceleration.csv"
    with csv_path.open("w", newline="", encoding="utf-8") as handle:
        writer = csv.DictWriter(handle, fieldnames=["config", "rank", "device", "world_size", "parameter_count", "phase",
                                                    "mean_ms", "std_ms", "peak_memory_mb"])
        writer.writeheader()
        for r in results:
            for phase in PHASES:
                stat: PhaseStats = getattr(r, phase)
                writer.writerow({"config": r.config, "rank": r.rank, "device": r.device, "world_size": r.world_size,
                                 "parameter_count": r.parameter_count, "phase": phase, "mean_ms": stat.mean_ms,
                                 "std_ms": stat.std_ms, "peak_memory_mb": stat.peak_memory_mb})
    first = [r for r in results if r.rank == 0]
    labels = [r.config for r in first]
    paths = {"json": str(json_path), "csv": str(csv_path)}
    times = {phase: [getattr(r, phase).mean_ms for r in first] for phase in ("forward", "backward", "optimizer")}
    memory = {"peak": [r.total.peak_memory_mb for r in first]}
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        fig, axes = plt.subplots(1, 2, figsize=(12, 4.5))
        x = range(len(labels))
        for i, (phase, values) in enumerate(times.items()):
            axes[0].bar([v + 0.25 * i for v in x], values, width=0.25, label=phase)
        axes[0].set_xticks([v + 0.25 for v in x], labels, rotation=15)
        axes[0].set_ylabel("ms per step")
        axes[0].legend()
        axes[1].bar(list(x), memory["peak"])
        axes[1].set_xticks(list(x), labels, rotation=15)
        axes[1].set_ylabel("peak allocated MiB")
        fig.tight_layout()
        figure = out / "benchmark_acceleration.png"
        fig.savefig(figure, dpi=120)
        plt.close(fig)
        paths["figure"] = str(figure)
    except ImportError:
        _bars_svg(out / "benchmark_time.svg", "time per step", labels, times, "ms")
        _bars_svg(out / "benchmark_memory.svg", "peak allocated memory", labels, memory, "MiB")
        paths["figure"] = str(out / "benchmark_time.svg")
    return paths


def print_summary(results: list[BenchmarkResult]) -> None:
    print("\n" + "=" * 80 + "\nBENCHMARK SUMMARY\n" + "=" * 80)
    for config in CONFIGS:
        for r in (x for x in results if x.config == config and x.rank == 0):
            print(f"\n{config.upper().replace('_', ' ')} ({r.device}, {r.world_size} rank(s), {r.tokens_per_second:,.0f} tokens/s):")
            for phase in PHASES:
                stat = getattr(r, phase)
                print(f"  {phase.capitalize():10s} {stat.mean_ms:9.2f} ms  |  Peak Memory: {stat.peak_memory_mb:9.2f} MB")


def main(argv=None) -> dict:
    args = parse_args(argv)
    results: list[BenchmarkResult] = []
    for config in args.configs:
        if "fsdp" in config and args.world_size < 2:
            print(f"[{config}] runs unsharded: --world-size is 1")
        print(f"[{config}] ...", flush=True)
        results.extend(run_config(args, config))
    paths = write_outputs(args, results)
    print_summary(results)
    print("\nwritten:", ", ".join(paths.values()))
    return {"results": [asdict(r) for r in results], **paths}


if __name__ == "__main__":
    main()
