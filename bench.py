"""Benchmarks of record. Headline: training tokens/s of the dense 1.3B-class decoder (24 layers, d_model 2048,
16 heads x 128, 8 KV heads, SwiGLU 5632, vocab 32000, seq 4096, global batch 32 sequences, bf16 with fp32 AdamW
master weights, no activation checkpointing) on N GPUs of one node, tensor-parallel over N.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...        # the unmodified reference from baseline/_ref

Rank 0 prints one JSON line. ``value`` is device-timed (CUDA events, max over ranks) with the step's token batches
already resident on the GPU; ``e2e`` times the same steps through the training API with every micro-batch copied
from pinned host memory and the loss read back each step.

After the headline workload the same invocation measures the other workloads of the benchmark suite as short runs and
attaches them under ``secondary`` of the same JSON line (``--no-secondary`` skips them):

    dense1p3b_mha16   the headline model with 16 KV heads, the shape the reference arm is limited to
    dense8b_fsdp      8B decoder, fully sharded over N, micro-batch 2 x 8192 per GPU, accumulation 4, per-layer recompute
    moe64e_ep         64-expert top-6 MoE (+2 shared experts), expert parallel over N inside the sharded runtime
    serve_8b          8B decoder behind the paged-KV engine, tensor-parallel over N (bench_serve.py --suite)

Each secondary workload runs in child processes of its own (one per rank, own rendezvous port, a time limit), started
after this process has released the GPU, so a failure there cannot take the headline number with it. ``--workload``
runs one of them directly. The reference arm does the same with the workloads the reference can express
(``dense8b_fsdp`` with its own FSDP wrapper, ``serve_8b`` with its ``generate()`` on a few requests).
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MODEL = {"name": "dense_1p3b", "context_length": 4096, "d_model": 2048, "num_layers": 24, "num_heads": 16,
         "num_kv_heads": 8, "d_ff": 5632, "position_encoding": {"type": "rope", "theta": 10000.0},
         "init": {"type": "normal", "std": 0.02}}
VOCAB = 32000
GLOBAL_BATCH = 32
SEQ = 4096
METRIC = "train tokens/sec"

DENSE_8B = {"name": "dense_8b", "context_length": 8192, "d_model": 4096, "num_layers": 32, "num_heads": 32,
            "num_kv_heads": 8, "d_ff": 14336, "position_encoding": {"type": "rope", "theta": 500000.0},
            "init": {"type": "normal", "std": 0.02}}
MOE_64E = {"name": "moe_64e", "context_length": 4096, "d_model": 2048, "num_layers": 24, "num_heads": 16,
           "num_kv_heads": 4, "d_ff": 1408,
           "moe": {"num_experts": 64, "top_k": 6, "shared_experts": 2, "d_ff": 1408, "aux_loss_coef": 0.01,
                   "capacity_factor": 1.25},
           "position_encoding": {"type": "rope", "theta": 10000.0}, "init": {"type": "normal", "std": 0.02}}

# bytes of training state per parameter: bf16 working copy, fp32 master, gradient and two moments
STATE_BYTES_PER_PARAM = 18
GPU_BYTES = 180e9


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--micro-batch", type=int, default=0, help="sequences per micro-batch (0 = pick by N)")
    ap.add_argument("--layers", type=int, default=0, help="debug only: override the layer count (marks the run invalid)")
    ap.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    ap.add_argument("--seq", type=int, default=SEQ)
    ap.add_argument("--kv-heads", type=int, default=0, help="dense1p3b_tp only: KV heads (16 = the reference arm's shape)")
    ap.add_argument("--workload", default="dense1p3b_tp",
                    choices=["dense1p3b_tp", "dense8b_fsdp", "moe64e_ep", "serve_8b"],
                    help="dense8b_fsdp: 8B, FSDP over N, micro-batch 2 x 8192 per GPU, accumulation 4, per-layer "
                         "checkpointing; moe64e_ep: 64-expert top-6 MoE, EP = N with FSDP, 8 x 4096 per GPU; "
                         "serve_8b: the serving suite of bench_serve.py")
    ap.add_argument("--no-secondary", action="store_true", help="headline workload only")
    ap.add_argument("--child", action="store_true", help=argparse.SUPPRESS)
    return ap.parse_args()


def baseline_value():
    try:
        published = json.loads((ROOT / "BASELINE.json").read_text()).get("published") or {}
        for key in ("train_tokens_per_sec", "tokens_per_sec", "value"):
            if key in published:
                return float(published[key])
    except Exception:
        pass
    return None


def emit(payload: dict) -> None:
    print(json.dumps(payload), flush=True)


def synthetic_batches(global_batch: int, seq: int, micro: int, count: int, pin: bool):
    """``count`` steps of uniform-random token ids (seed 0): list[step] of list[micro-batch] of int64
    ``[micro, seq + 1]`` host tensors."""
    import torch

    gen = torch.Generator().manual_seed(0)
    steps = []
    for _ in range(count):
        tokens = torch.randint(0, VOCAB, (global_batch, seq + 1), generator=gen, dtype=torch.int64)
        pieces = [tokens[i:i + micro].contiguous() for i in range(0, global_batch, micro)]
        steps.append([p.pin_memory() if pin else p for p in pieces])
    return steps


# =============================================================================================== ours
def run_ours(args) -> dict | None:
    import torch
    import torch.distributed as dist

    from ajllm_b200.models import build_model
    from ajllm_b200.ops import native
    from ajllm_b200.parallel import ParallelMesh, init_distributed, tp_optimizer_classes
    from ajllm_b200.parallel.contexts import make_tensor_parallel, tp_backend
    from ajllm_b200.training import FlatAdamW, optimizer_step
    from ajllm_b200.utils.timing import ClockSampler, max_over_ranks

    rank, world, device = init_distributed("cuda")
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE is {world}; launch with torch.distributed.run")
    assert native.available(), "native kernel library missing: run python -m ajllm_b200.build"
    torch.manual_seed(0)
    config = dict(MODEL)
    config["context_length"] = args.seq
    if args.layers:
        config["num_layers"] = args.layers
    if args.kv_heads:
        config["num_kv_heads"] = args.kv_heads
    tp = None
    classes = None
    if world > 1:
        tp = make_tensor_parallel(ParallelMesh(tp=world).tp, device)
        classes = tp_optimizer_classes(tp)
    with torch.device(device):
        model = build_model(config, VOCAB, tp=tp)
    model = model.to(device=device, dtype=torch.bfloat16)
    # sequences per micro-batch, measured: one GPU runs 16 (1 % faster than 8; the 16-KV-head variant keeps 8, its
    # activations are larger), two GPUs 16 (32 halves the throughput: the gathered activations kept for the backward
    # pass no longer fit beside the rest), four 16, eight 32; with two micro-batches in flight (model.interleave,
    # opt-in) the batch of 32 is cut into at least two
    micro = args.micro_batch or {1: 16 if not args.kv_heads or args.kv_heads == 8 else 8, 2: 16, 4: 16,
                                 8: 32 if model.interleave == 1 else 16}.get(world, 8)
    micro = min(micro, args.global_batch)
    accumulation = args.global_batch // micro
    optimizer = FlatAdamW(model, learning_rate=3e-4, betas=(0.9, 0.95), epsilon=1e-8, weight_decay=0.1, classes=classes)
    params = sum(p.numel() for p in model.parameters())

    total_steps = args.warmup + args.steps
    host_steps = synthetic_batches(args.global_batch, args.seq, micro, total_steps, pin=True)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def device_feed(step_batches):
        staged = [b.to(device, non_blocking=True) for b in step_batches]
        it = iter(staged)

        def next_batch():
            t = next(it)
            return t[:, :-1], t[:, 1:]
        return next_batch

    # ---- pass A: device-timed, batches resident on the GPU
    for s in range(args.warmup):
        optimizer_step(model, optimizer, device_feed(host_steps[s]), accumulation, 1.0)
    timed = host_steps[args.warmup:]
    feeds = [device_feed(b) for b in timed]
    barrier()
    sampler = ClockSampler(device.index or 0).start()
    launches0 = native.launch_count
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for feed in feeds:
        loss, norm = optimizer_step(model, optimizer, feed, accumulation, 1.0)
    end.record()
    barrier()
    clocks = sampler.stop()
    launches = native.launch_count - launches0
    ms = max_over_ranks(begin.elapsed_time(end), device)
    final_loss = float(loss.detach()) * (world if tp is not None else 1)
    tokens = args.global_batch * args.seq * args.steps
    value = tokens / (ms / 1e3)

    # ---- pass B: end to end (pinned host -> device every micro-batch, loss read back every step)
    copy_stream = torch.cuda.Stream(device=device)

    def host_feed(step_batches):
        it = iter(step_batches)

        def next_batch():
            with torch.cuda.stream(copy_stream):
                t = next(it).to(device, non_blocking=True)
            torch.cuda.current_stream().wait_stream(copy_stream)
            t.record_stream(torch.cuda.current_stream())
            return t[:, :-1], t[:, 1:]
        return next_batch

    barrier()
    t0 = time.perf_counter()
    begin2, end2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin2.record()
    readback = []
    for step_batches in timed:
        loss, norm = optimizer_step(model, optimizer, host_feed(step_batches), accumulation, 1.0)
        readback.append(float(loss.detach()))          # device -> host read of the step's result
    end2.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    e2e_ms = max_over_ranks(max(begin2.elapsed_time(end2), wall_ms), device)
    h2d = args.global_batch * (args.seq + 1) * 8
    status = native.lib().ajb_check_status()
    overlap = getattr(model, "overlap_description", None)

    payload = None
    if rank == 0:
        base = baseline_value()
        kv = config["num_kv_heads"]
        payload = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": (value / base) if base else None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": f"dense-1.3B (24L d2048 16h/{kv}kv hd128 ffn5632 vocab32000)", "params_on_rank": params,
                       "global_batch": args.global_batch, "seq_len": args.seq, "micro_batch": micro,
                       "grad_accumulation": accumulation, "parallelism": f"tp{world}",
                       "tp_backend": tp_backend(tp), "overlap": overlap,
                       "optimizer": "AdamW fp32 master, global-norm clip 1.0", "activation_checkpointing": "off",
                       "l2": "inputs larger than L2 (multi-GB working set per step)",
                       "layers_override": args.layers or None},
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"),
                       "reasons": clocks.get("reasons"), "power_w_max": clocks.get("power_w_max")},
            "e2e": {"value": tokens / (e2e_ms / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": 4, "ms_per_step": e2e_ms / args.steps},
            "gpu_launches": launches, "final_loss": final_loss, "kernel_status": status,
            "valid": not args.layers and args.global_batch == GLOBAL_BATCH and args.seq == SEQ,
        }
    # release the GPU before any secondary workload starts in a child process
    del model, optimizer, feeds, loss, norm
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    torch.cuda.empty_cache()
    return payload


def run_sharded(args) -> dict | None:
    """Weak-scaling workloads on the fully-sharded runtime (8B dense; 64-expert MoE with expert parallelism)."""
    import torch
    import torch.distributed as dist

    from ajllm_b200.models import build_model
    from ajllm_b200.ops import native
    from ajllm_b200.parallel import ParallelMesh, init_distributed
    from ajllm_b200.parallel.contexts import expert_exchange_backend, make_expert_parallel
    from ajllm_b200.training import FlatAdamW, optimizer_step
    from ajllm_b200.utils.timing import ClockSampler, max_over_ranks

    rank, world, device = init_distributed("cuda")
    moe = args.workload == "moe64e_ep"
    config = dict(MOE_64E if moe else DENSE_8B)
    vocab = 32000 if moe else 128256
    if args.layers:
        config["num_layers"] = args.layers
    seq = config["context_length"]
    per_gpu_batch, accumulation = (8, 1) if moe else (2, 4)
    micro = args.micro_batch or (4 if moe else 2)
    accumulation = accumulation * (per_gpu_batch // micro)
    torch.manual_seed(0)
    ep = None
    mesh = None
    if world > 1:
        mesh = ParallelMesh(tp=1, fsdp=world, ep=world if moe else 1)
        if moe:
            ep = make_expert_parallel(mesh.ep, device)
    with torch.device(device):
        model = build_model(config, vocab, ep=ep, activation_checkpointing="layer" if world == 1 else "none")
    model = model.to(device=device, dtype=torch.bfloat16)
    params_local = sum(p.numel() for p in model.parameters())
    if world > 1:
        from ajllm_b200.parallel.fsdp import ShardedDataParallel
        model = ShardedDataParallel(model, mesh.dp.group, learning_rate=3e-4, betas=(0.9, 0.95), epsilon=1e-8,
                                    weight_decay=0.1)
        optimizer = model.optimizer
    else:
        optimizer = FlatAdamW(model, learning_rate=3e-4, betas=(0.9, 0.95), epsilon=1e-8, weight_decay=0.1)
    gen = torch.Generator().manual_seed(rank)
    total_steps = args.warmup + args.steps
    host = [[torch.randint(0, vocab, (micro, seq + 1), generator=gen).pin_memory() for _ in range(accumulation)]
            for _ in range(total_steps)]

    def feed(step_batches):
        it = iter(step_batches)

        def next_batch():
            t = next(it).to(device, non_blocking=True)
            return t[:, :-1], t[:, 1:]
        return next_batch

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for s in range(args.warmup):
        optimizer_step(model, optimizer, feed(host[s]), accumulation, 1.0)
    barrier()
    sampler = ClockSampler(device.index or 0).start()
    launches0 = native.launch_count
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    begin.record()
    losses = []
    for s in range(args.warmup, total_steps):
        loss, norm = optimizer_step(model, optimizer, feed(host[s]), accumulation, 1.0)
        losses.append(float(loss.detach()))
    end.record()
    barrier()
    wall_ms = (time.perf_counter() - t0) * 1e3
    clocks = sampler.stop()
    ms = max_over_ranks(begin.elapsed_time(end), device)
    wall_ms = max_over_ranks(wall_ms, device)
    tokens = world * per_gpu_batch * (4 if not moe else 1) * seq * args.steps
    peak = torch.cuda.max_memory_allocated(device) / 2**30
    payload = None
    if rank == 0:
        payload = {
            "metric": METRIC, "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "impl": "ours",
            "config": {"model": config["name"], "params_on_rank": params_local, "per_gpu_batch": per_gpu_batch,
                       "seq_len": seq, "micro_batch": micro, "grad_accumulation": accumulation,
                       "parallelism": (f"ep{world} x fsdp{world}" if moe else f"fsdp{world}") if world > 1 else "single",
                       "expert_exchange": expert_exchange_backend(ep) if moe else None,
                       "activation_checkpointing": "per layer", "layers_override": args.layers or None,
                       "timed_region": "includes the pinned-host to device copy of every micro-batch and the loss read-back"},
            "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons")},
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": accumulation * micro * (seq + 1) * 8, "d2h_bytes_per_step": 4},
            "gpu_launches": native.launch_count - launches0, "final_loss": losses[-1], "peak_memory_gib": peak,
            "kernel_status": native.lib().ajb_check_status(),
        }
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return payload


# =============================================================================================== reference
def _reference_imports():
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "ajllm" / "__init__.py").is_file():
        return None, "baseline/_ref holds no reference install"
    sys.path.insert(0, str(ref_root))
    try:
        import ajllm.modeling.factory  # noqa: F401
        import ajllm.training.distributed  # noqa: F401
    except Exception as error:  # noqa: BLE001
        return None, f"reference import failed: {type(error).__name__}: {error}"[:300]
    return ref_root, None


def _is_oom(error: BaseException) -> bool:
    import torch
    return isinstance(error, torch.cuda.OutOfMemoryError) or "out of memory" in str(error).lower()


def run_reference(args) -> dict | None:
    """The unmodified reference driven through its own public API: ``build_model(use_flash_attention=True)`` (its
    Triton kernels), ``FullyShardedDataParallel(bf16)``, ``cross_entropy``, ``clip_gradients``, ``AdamW``. It has no
    gradient accumulation, so it is given the largest micro-batch that fits (fewest optimizer passes per batch)."""
    _, problem = _reference_imports()
    if problem:
        return {"impl": "reference", "unavailable": problem}
    import torch
    import torch.distributed as dist
    from ajllm.modeling.factory import build_model
    from ajllm.training.distributed import FullyShardedDataParallel
    from ajllm.training.losses import cross_entropy
    from ajllm.training.optimizers import AdamW
    from ajllm.training.trainer import clip_gradients

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    big = args.workload == "dense8b_fsdp"
    if big:
        # the 8B shape as the reference can express it: 32 full heads (8.84 B parameters), every rank 2 x 8192 tokens
        # per optimizer step (it cannot accumulate the 4 micro-batches of the configuration)
        config = {"name": "dense_8b_mha", "context_length": 8192, "d_model": 4096, "num_layers": args.layers or 32,
                  "num_heads": 32, "d_ff": 14336, "position_encoding": {"type": "rope", "theta": 500000.0}}
        vocab, seq, global_batch = 128256, 8192, 2 * world
        candidates = [args.micro_batch] if args.micro_batch else [2, 1]
    else:
        # the reference has no grouped KV heads: same shape with 16 full heads (1.364 B parameters)
        config = {"name": "dense_1p3b_mha", "context_length": args.seq, "d_model": 2048, "num_layers": args.layers or 24,
                  "num_heads": 16, "d_ff": 5632, "position_encoding": {"type": "rope", "theta": 10000.0}}
        vocab, seq, global_batch = VOCAB, args.seq, args.global_batch
        per_rank = global_batch // world
        candidates = [args.micro_batch] if args.micro_batch else [m for m in (16, 8, 4, 2, 1) if m <= per_rank]
    total_steps = args.warmup + args.steps
    tried: list[int] = []

    def attempt(micro: int) -> dict:
        torch.manual_seed(0)
        model = build_model(config, vocab, use_flash_attention=True).to(device)
        model = FullyShardedDataParallel(model, compute_dtype=torch.bfloat16)
        optimizer = AdamW(model.parameters(), learning_rate=3e-4, betas=(0.9, 0.95), epsilon=1e-8, weight_decay=0.1)
        gen = torch.Generator().manual_seed(0)
        host_steps = []
        for _ in range(total_steps):
            tokens = torch.randint(0, vocab, (global_batch, seq + 1), generator=gen, dtype=torch.int64)
            pieces = [tokens[i:i + micro].contiguous().pin_memory() for i in range(0, global_batch, micro)]
            host_steps.append([b for i, b in enumerate(pieces) if i % world == rank])

        def one_step(step_batches):
            last = None
            for batch in step_batches:
                t = batch.to(device, non_blocking=True)
                logits = model(t[:, :-1])
                loss = cross_entropy(logits, t[:, 1:])
                optimizer.zero_grad(set_to_none=True)
                loss.backward()
                model.finish_gradient_synchronization()
                clip_gradients(model.parameters(), 1.0)
                optimizer.step()
                last = loss
            return last

        def barrier():
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        for s in range(args.warmup):
            one_step(host_steps[s])
        barrier()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        begin.record()
        for s in range(args.warmup, total_steps):
            loss = one_step(host_steps[s])
            float(loss.detach())
        end.record()
        barrier()
        wall_ms = (time.perf_counter() - t0) * 1e3
        ms = begin.elapsed_time(end)
        if world > 1:
            box = torch.tensor([ms, wall_ms], device=device, dtype=torch.float64)
            dist.all_reduce(box, op=dist.ReduceOp.MAX)
            ms, wall_ms = float(box[0]), float(box[1])
        tokens = global_batch * seq * args.steps
        return {
            "metric": METRIC, "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True,
            "scaling": "weak" if big else "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "impl": "reference",
            "config": {"model": ("dense-8B as the reference can express it: MHA 32 heads (8.84B params)" if big else
                                 "dense-1.3B as the reference can express it: MHA 16 heads (1.364B params)"),
                       "global_batch": global_batch, "seq_len": seq, "micro_batch": micro,
                       "micro_batches_tried": list(tried),
                       "parallelism": f"reference FSDP over {world} (its only parallelism), bf16 compute, Triton flash attention",
                       "note": "no gradient accumulation in the reference: optimizer step per micro-batch; "
                               "the largest micro-batch that fits is used"},
            "e2e": {"value": tokens / (wall_ms / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": global_batch * (seq + 1) * 8, "d2h_bytes_per_step": 4},
            "peak_memory_gib": torch.cuda.max_memory_allocated(device) / 2**30,
        }

    payload, last_error = None, None
    for micro in candidates:
        tried.append(micro)
        failed = 0
        try:
            payload = attempt(micro)
        except Exception as error:  # noqa: BLE001 - out of memory moves on to a smaller micro-batch
            # keep the text only: the exception's traceback would pin the failed attempt's tensors
            last_error = f"{type(error).__name__}: {error}"
            failed = 1 if _is_oom(error) else 2
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        # every rank must take the same branch: a rank that ran out of memory stops the others too
        if world > 1:
            flag = torch.tensor([failed], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MAX)
            failed = int(flag)
        if failed == 0:
            break
        payload = None
        if failed == 2:
            break
    if payload is None:
        why = last_error if last_error is not None else "a peer rank failed"
        payload = {"impl": "reference", "unavailable": f"reference run failed (micro-batches tried {tried}): {why}"[:400]}
    if world > 1 and dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()
    torch.cuda.empty_cache()
    return payload if rank == 0 else None


# =============================================================================================== secondary workloads
def _fits(params: float, world: int, what: str) -> str | None:
    need = params * STATE_BYTES_PER_PARAM / world
    if need > 0.8 * GPU_BYTES:
        return (f"skipped at {world} GPU(s): {what} holds {params / 1e9:.1f} B parameters x {STATE_BYTES_PER_PARAM} bytes of "
                f"training state = {need / 1e9:.0f} GB per GPU")
    return None


def _child(script: str, extra: list[str], port_offset: int, limit_s: float) -> dict:
    """Run ``script`` in a child of this rank (same RANK / WORLD_SIZE, a rendezvous port of its own) and return the
    JSON line its rank 0 printed. The child is killed by its exact pid when it exceeds ``limit_s``."""
    env = dict(os.environ)
    if "MASTER_PORT" in env:
        env["MASTER_PORT"] = str(int(env["MASTER_PORT"]) + port_offset)
    env.setdefault("MASTER_ADDR", "127.0.0.1")
    # the child hosts its own rendezvous store instead of joining the launcher's, and gives up quickly on a peer
    # that never arrives
    env.pop("TORCHELASTIC_USE_AGENT_STORE", None)
    env.setdefault("AJB_DIST_TIMEOUT_S", "180")
    rank = int(env.get("RANK", "0"))
    with tempfile.NamedTemporaryFile("w+", suffix=f".rank{rank}.log", delete=False) as log:
        proc = subprocess.Popen([sys.executable, str(ROOT / script), *extra], stdout=log, stderr=subprocess.STDOUT,
                                env=env, cwd=str(ROOT))
        try:
            code = proc.wait(timeout=limit_s)
        except subprocess.TimeoutExpired:
            proc.kill()
            proc.wait()
            code = "time limit"
        log.seek(0)
        text = log.read()
    os.unlink(log.name)
    for line in reversed(text.splitlines()):
        line = line.strip()
        if line.startswith("{") and line.endswith("}"):
            try:
                return json.loads(line)
            except ValueError:
                continue
    first = next((line.strip() for line in text.splitlines() if "Error" in line or "error:" in line), "")
    return {"error": f"no result (exit {code}): {first[:300]} ... " + text[-300:].replace("\n", " | ")}


SECONDARY_BUDGET_S = 480.0       # no further secondary workload starts once this much time has gone into them


def run_secondary(args, impl: str) -> dict:
    world = args.gpus
    common = ["--gpus", str(world), "--child", "--no-secondary", "--impl", impl]
    out: dict = {}
    started = time.perf_counter()

    rank = int(os.environ.get("RANK", "0"))
    tag = f'{os.environ.get("TORCHELASTIC_RUN_ID", "single")}_{os.environ.get("MASTER_PORT", "0")}'

    def child(name: str, script: str, extra: list[str], port_offset: int, limit_s: float) -> None:
        # rank 0 decides whether there is time left and tells the other ranks of the node through a file, so that
        # either every rank starts its child or none does
        note = Path(tempfile.gettempdir()) / f"ajb_bench_{tag}_{impl}_{name}.go"
        if rank == 0:
            left = SECONDARY_BUDGET_S - (time.perf_counter() - started)
            go = left >= 45.0
            note.write_text(f"{int(go)} {max(60.0, min(limit_s, left + 60.0)):.0f}")
        else:
            waited = 0.0
            while not note.exists() and waited < 90.0:
                time.sleep(0.2)
                waited += 0.2
        try:
            flag, limit = note.read_text().split()
            go, limit_s = flag == "1", float(limit)
        except (OSError, ValueError):
            go = False
        if not go:
            out[name] = {"skipped": "the time set aside for the secondary workloads of this run was used up"}
        else:
            out[name] = _child(script, extra, port_offset, limit_s)
        if rank == 0:
            time.sleep(1.0)                 # the other ranks have read the note by now
            note.unlink(missing_ok=True)

    if impl == "ours":
        child("serve_8b", "bench_serve.py", ["--gpus", str(world), "--suite"], 17, 300)
        skip = _fits(8.03e9, world, "the 8B decoder")
        if skip:
            out["dense8b_fsdp"] = {"skipped": skip}
        else:
            child("dense8b_fsdp", "bench.py", [*common, "--workload", "dense8b_fsdp", "--steps", "2", "--warmup", "3"], 13, 300)
        skip = _fits(13.9e9, world, "the 64-expert model")
        if skip:
            out["moe64e_ep"] = {"skipped": skip}
        else:
            child("moe64e_ep", "bench.py", [*common, "--workload", "moe64e_ep", "--steps", "3", "--warmup", "3"], 15, 240)
        child("dense1p3b_mha16", "bench.py", [*common, "--workload", "dense1p3b_tp", "--kv-heads", "16", "--steps", "3",
                                             "--warmup", "3"], 11, 200)
    else:
        child("serve_8b", "bench_serve.py", ["--gpus", str(world), "--impl", "reference", "--requests", "3"], 17, 300)
        child("dense8b_fsdp", "bench.py", [*common, "--workload", "dense8b_fsdp", "--steps", "2", "--warmup", "3"], 13, 300)
        out["moe64e_ep"] = {"impl": "reference", "unavailable": "the reference has no mixture-of-experts layer and no expert parallelism"}
    return out


def main() -> None:
    args = parse_args()
    if args.workload == "serve_8b":
        extra = ["--gpus", str(args.gpus), "--suite"] + (["--impl", "reference", "--requests", "3"] if args.impl == "reference" else [])
        os.execv(sys.executable, [sys.executable, str(ROOT / "bench_serve.py"), *extra])
    if args.impl == "reference":
        payload = run_reference(args)
    elif args.workload != "dense1p3b_tp":
        payload = run_sharded(args)
    else:
        payload = run_ours(args)
    rank = int(os.environ.get("RANK", "0"))
    headline = args.workload == "dense1p3b_tp" and not args.child
    if headline and not args.no_secondary and os.environ.get("AJB_BENCH_SECONDARY", "1") != "0":
        secondary = run_secondary(args, args.impl)          # every rank starts its children; rank 0 keeps the results
        if payload is not None:
            payload["secondary"] = secondary
    if rank == 0 and payload is not None:
        emit(payload)


if __name__ == "__main__":
    main()
