"""Serving benchmark: output tokens/s of the 8B-class decoder (32 layers, d_model 4096, 32 heads x 128,
8 KV heads, SwiGLU 14336, vocab 128256) behind the paged-KV continuous-batching engine, tensor-parallel
over N GPUs. Requests: prompt lengths uniform in [128, 2048], output lengths uniform in [64, 512], uniform
random token ids (seed 0), at most 256 concurrent sequences, random-init bf16 weights.

    python bench_serve.py --gpus 1 --requests 256
    python -m torch.distributed.run --nproc-per-node 8 ... bench_serve.py --gpus 8 --requests 1024 \
        [--quantization fp8] [--speculative 4] [--temperature 1.0]
    python bench_serve.py --suite                            # all variants, one JSON line (what bench.py attaches)
    python bench_serve.py --impl reference --requests 3      # the reference's generate(): batch 1, no KV cache

Rank 0 prints one JSON line; throughput is generated tokens divided by the wall time of the whole run
(submission to last token), bracketed by device synchronisation, max over ranks.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

MODEL = {"name": "dense_8b", "context_length": 4096, "d_model": 4096, "num_layers": 32, "num_heads": 32,
         "num_kv_heads": 8, "d_ff": 14336, "position_encoding": {"type": "rope", "theta": 500000.0},
         "init": {"type": "normal", "std": 0.02}}
VOCAB = 128256


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--requests", type=int, default=256)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--max-batched-tokens", type=int, default=8192)
    ap.add_argument("--quantization", default=None)
    ap.add_argument("--speculative", type=int, default=0, help="k draft tokens per step (2-layer random-init draft)")
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--layers", type=int, default=0)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--self-draft", action="store_true", help="with --speculative: the draft is the target's first 2 layers")
    ap.add_argument("--decode-steps", type=int, default=0,
                    help="instead of the request mix: fill --max-num-seqs sequences of --context tokens, then time this "
                         "many pure decoding steps (ms per step on the device and on the host clock)")
    ap.add_argument("--context", type=int, default=1280, help="with --decode-steps: prompt tokens per sequence")
    ap.add_argument("--suite", action="store_true",
                    help="bf16 greedy on --requests requests, then shorter fp8 / speculative variants, in one JSON line")
    return ap.parse_args()


def make_requests(count: int):
    import numpy as np
    rng = np.random.default_rng(0)
    prompts = [rng.integers(0, VOCAB, size=int(rng.integers(128, 2049))).tolist() for _ in range(count)]
    outputs = [int(rng.integers(64, 513)) for _ in range(count)]
    return prompts, outputs


def _self_draft(model, config, layers: int = 2):
    """A draft that IS the first ``layers`` blocks of the target (shared embeddings, norm and head): no extra weights,
    and its proposals follow the target closely because both read the same residual stream."""
    import torch

    from ajllm_b200.models import build_model

    with torch.device("meta"):
        draft = build_model({**config, "num_layers": layers}, VOCAB, tp=model.tp)
    draft.token_embeddings = model.token_embeddings
    draft.position_embeddings = model.position_embeddings
    draft.layers = torch.nn.ModuleList(list(model.layers[:layers]))
    draft.final_norm = model.final_norm
    draft.lm_head = model.lm_head
    return draft


def _decode_steps(args, model, device, quantization=None):
    """Pure decoding: every sequence holds ``--context`` tokens, each timed step emits one token per sequence."""
    import numpy as np
    import torch

    from ajllm_b200.engine import LLMEngine, SamplingParams

    seqs, steps = args.max_num_seqs, args.decode_steps
    # sequences admitted first keep decoding while the others are still prefilled: nobody may finish before the end
    fill_steps = -(-seqs * args.context // args.max_batched_tokens) + 8
    budget = fill_steps + steps + 16
    blocks = (seqs * (args.context + budget + 32)) // 16
    engine = LLMEngine(model, block_size=16, num_blocks=blocks, max_num_seqs=seqs,
                       max_batched_tokens=args.max_batched_tokens, quantization=quantization, seed=0)
    rng = np.random.default_rng(0)
    for _ in range(seqs):
        engine.add_request(rng.integers(0, VOCAB, size=args.context).tolist(), SamplingParams(budget, 0.0, None, None))
    for _ in range(fill_steps):
        engine.step()
    if len(engine.scheduler.running) != seqs or any(seq.computed < args.context for seq in engine.scheduler.running):
        raise RuntimeError("the sequences were not all prefilled within the expected number of steps")
    for _ in range(3):
        engine.step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.profiler.start()          # a profiler started with --profile-from-start off sees only the timed steps
    t0 = time.perf_counter()
    begin.record()
    for _ in range(steps):
        engine.step()
    end.record()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    host_ms = (time.perf_counter() - t0) * 1e3 / steps
    return {"metric": "decode step", "sequences": seqs, "context": args.context, "steps": steps,
            "dtype": quantization or "bf16", "ms_per_step_device": begin.elapsed_time(end) / steps,
            "ms_per_step_host": host_ms, "tokens_per_s": seqs / host_ms * 1e3}


def _one_run(args, model, config, tp, device, rank, world, *, requests, quantization=None, speculative=0,
             temperature=0.0, self_draft=False):
    import torch
    import torch.distributed as dist

    from ajllm_b200.engine import LLMEngine, SamplingParams
    from ajllm_b200.models import build_model
    from ajllm_b200.ops import native
    from ajllm_b200.parallel.contexts import tp_backend
    from ajllm_b200.utils.timing import ClockSampler

    draft = None
    if speculative:
        if self_draft:
            draft = _self_draft(model, config)
        else:
            torch.manual_seed(1)
            with torch.device(device):
                draft = build_model({**config, "num_layers": 2}, VOCAB, tp=tp).to(dtype=torch.bfloat16)
    prompts, outputs = make_requests(requests)
    blocks = (args.max_num_seqs * (2048 + 512 + 64)) // 16
    engine = LLMEngine(model, block_size=16, num_blocks=blocks, max_num_seqs=args.max_num_seqs,
                       max_batched_tokens=args.max_batched_tokens, quantization=quantization, draft_model=draft,
                       num_speculative_tokens=speculative or 4, seed=0)
    params = [SamplingParams(n, temperature, None, None, seed=i) for i, n in enumerate(outputs)]
    # warm-up: the decoding graphs of every batch-size bucket, then a few short requests through every code path
    engine.warm_up()
    engine.generate([p[:160] for p in prompts[:4]], [SamplingParams(8, temperature, None) for _ in range(4)])
    engine.stats = type(engine.stats)()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches0 = native.launch_count
    sampler = ClockSampler(device.index or 0).start()
    t0 = time.perf_counter()
    results = engine.generate(prompts, params)
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    clocks = sampler.stop()
    if world > 1:
        box = torch.tensor([elapsed], device=device, dtype=torch.float64)
        dist.all_reduce(box, op=dist.ReduceOp.MAX)
        elapsed = float(box)
    generated = sum(len(r.output) for r in results)
    prompt_tokens = sum(len(p) for p in prompts)
    steps = max(1, engine.stats.steps)
    record = {
        "metric": "serve output tokens/sec", "value": generated / elapsed, "unit": "tokens/s", "n_gpus": world,
        "impl": "ours", "dtype": "bf16" if not quantization else quantization, "data": "synthetic",
        "higher_is_better": True,
        "config": {"model": "dense-8B (32L d4096 32h/8kv hd128 ffn14336 vocab128256)", "requests": requests,
                   "prompt_len": "U[128,2048]", "output_len": "U[64,512]", "max_num_seqs": args.max_num_seqs,
                   "parallelism": f"tp{world}", "tp_backend": tp_backend(tp), "speculative_k": speculative,
                   "draft": ("first 2 layers of the target" if self_draft else "random-init 2-layer model") if speculative else None,
                   "temperature": temperature, "layers_override": args.layers or None,
                   "timing": "host wall clock from submission to the last token, device synchronised on both sides, "
                             "max over ranks; every step copies its token ids / block tables from the host and reads "
                             "the sampled tokens back"},
        "elapsed_s": elapsed, "output_tokens": generated, "prompt_tokens": prompt_tokens,
        "engine_steps": engine.stats.steps, "ms_per_step": elapsed * 1e3 / steps, "preemptions": engine.stats.preemptions,
        "draft_acceptance_rate": engine.stats.acceptance_rate if speculative else None,
        "clocks": {"sm_mhz": clocks.get("sm_mhz"), "sm_max_mhz": clocks.get("sm_max_mhz"), "reasons": clocks.get("reasons")},
        # the whole run is end to end: inputs start as host token lists, outputs end as host token lists
        "e2e": {"value": generated / elapsed, "unit": "tokens/s",
                "h2d_bytes_per_step": int((prompt_tokens + generated) * 8 * 4 / steps),
                "d2h_bytes_per_step": int(generated * 8 / steps)},
        "gpu_launches": native.launch_count - launches0, "kernel_status": native.lib().ajb_check_status(),
    }
    del engine, draft
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return record


def run_ours(args):
    import torch
    import torch.distributed as dist

    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ParallelMesh, init_distributed
    from ajllm_b200.parallel.contexts import make_tensor_parallel

    rank, world, device = init_distributed("cuda")
    tp = make_tensor_parallel(ParallelMesh(tp=world).tp, device, interleave=1) if world > 1 else None
    torch.manual_seed(0)
    config = dict(MODEL)
    if args.layers:
        config["num_layers"] = args.layers
    with torch.device(device):
        model = build_model(config, VOCAB, tp=tp).to(dtype=torch.bfloat16)
    run = lambda **kw: _one_run(args, model, config, tp, device, rank, world, **kw)   # noqa: E731
    if args.decode_steps:
        record = _decode_steps(args, model, device, args.quantization)
    elif not args.suite:
        record = run(requests=args.requests, quantization=args.quantization, speculative=args.speculative,
                     temperature=args.temperature, self_draft=args.self_draft)
    else:
        # the headline variant first, then the shorter ones; a variant that fails is reported, not fatal
        record = run(requests=args.requests)
        variants = {}
        small = max(16, args.requests // 4)
        for name, kw in (("fp8_greedy", dict(requests=args.requests // 2, quantization="fp8")),
                         ("bf16_spec4_greedy", dict(requests=small, speculative=4)),
                         ("bf16_spec4_t1", dict(requests=small, speculative=4, temperature=1.0))):
            try:
                full = run(**kw)
                variants[name] = {k: full[k] for k in ("value", "elapsed_s", "output_tokens", "engine_steps", "ms_per_step",
                                                       "draft_acceptance_rate", "gpu_launches", "kernel_status")}
                variants[name]["requests"] = kw["requests"]
            except Exception as error:  # noqa: BLE001
                variants[name] = {"error": f"{type(error).__name__}: {error}"[:300]}
                if world > 1:
                    break          # ranks may have diverged: stop here rather than wait on one another
        record["variants"] = variants
    if rank == 0:
        print(json.dumps(record), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_reference(args):
    """The reference's stock ``generate()`` (``ajllm/generation/generator.py:10-28``: one request at a time, the whole
    context re-run for every new token) on the first ``--requests`` requests of the workload; the first is the warm-up.
    It has one GPU's worth of parallelism, so under a multi-rank launch only rank 0 works."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    ref_root = ROOT / "baseline" / "_ref"
    if not (ref_root / "ajllm" / "__init__.py").is_file():
        print(json.dumps({"impl": "reference", "unavailable": "baseline/_ref holds no reference install"}))
        return
    sys.path.insert(0, str(ref_root))
    import torch
    from ajllm.generation.generator import generate
    from ajllm.modeling.factory import build_model

    device = torch.device("cuda", 0)
    torch.manual_seed(0)
    config = {"name": "dense_8b_mha", "context_length": 4096, "d_model": 4096, "num_layers": args.layers or 32,
              "num_heads": 32, "d_ff": 14336, "position_encoding": {"type": "rope", "theta": 500000.0}}
    try:
        with torch.device(device):
            model = build_model(config, VOCAB).to(dtype=torch.bfloat16)
        prompts, outputs = make_requests(args.requests)
        generated, t0 = 0, None
        for i, (p, n) in enumerate(zip(prompts, outputs)):
            if i == 1 or (i == 0 and len(prompts) == 1):
                torch.cuda.synchronize()
                t0, generated = time.perf_counter(), 0          # first request is the warm-up when there are several
            out = generate(model, torch.tensor(p, device=device), n, args.temperature, None, None)
            generated += out.numel() - len(p)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t0
        print(json.dumps({"metric": "serve output tokens/sec", "value": generated / elapsed, "unit": "tokens/s",
                          "n_gpus": 1, "impl": "reference", "dtype": "bf16", "data": "synthetic",
                          "higher_is_better": True,
                          "config": {"model": "dense-8B as the reference can express it: MHA, generate() batch 1, no KV cache",
                                     "requests_timed": max(1, len(prompts) - 1),
                                     "note": "tokens/s as measured on this subset of the request list"},
                          "elapsed_s": elapsed, "output_tokens": generated}))
    except Exception as error:  # noqa: BLE001
        print(json.dumps({"impl": "reference", "unavailable": f"{type(error).__name__}: {error}"[:300]}))


if __name__ == "__main__":
    a = parse_args()
    run_reference(a) if a.impl == "reference" else run_ours(a)
