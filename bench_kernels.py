"""Kernel microbenchmarks on one B200: the tcgen05 GEMM against cuBLAS on the layer shapes of the flagship
model, the attention kernels, the fused norm kernels, paged decode attention with and without the split over the keys,
the sampler, the block-scaled fp8 GEMM, and the gradient reduce-scatter kernel emulated on one GPU.

    python bench_kernels.py                      # everything, full-size shapes
    python bench_kernels.py --case flash --small # a small case (for a profiler capture)
    python bench_kernels.py --case decode        # decoding GEMMs (few rows) against cuBLAS, GB/s of weights

Timing: CUDA events around 10 launches after 3 warm-up launches; operands are larger than L2 for the GEMM
and norm cases. FLOP counts: 2 m n k for a GEMM; attention forward 4 B H T^2 d / 2 (causal), backward
2.5 times that (five products), whatever the kernel actually executes.
"""

from __future__ import annotations

import argparse
import math

import torch

from ajllm_b200 import ops
from ajllm_b200.ops import native


def timeit(fn, iters: int = 10, warmup: int = 3) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    return begin.elapsed_time(end) / iters


def gemm_case(dev, name, m, n, k, a_mn=False, b_mn=False, epilogue=0) -> None:
    a = torch.randn((k, m) if a_mn else (m, k), device=dev, dtype=torch.bfloat16)
    b = torch.randn((k, n) if b_mn else (n, k), device=dev, dtype=torch.bfloat16)
    out = torch.zeros(m, n, device=dev, dtype=torch.float32 if epilogue else torch.bfloat16)
    ours = timeit(lambda: ops.gemm(a, b, out, m, n, k, a_mn_major=a_mn, b_mn_major=b_mn, epilogue=epilogue))
    left, right = (a.t() if a_mn else a), (b if b_mn else b.t())
    cublas = timeit(lambda: torch.matmul(left, right))
    flops = 2 * m * n * k
    print(f"{name:24s} m{m} n{n} k{k}: ours {ours * 1e3:8.1f} us {flops / ours / 1e9:7.1f} TF | cuBLAS {cublas * 1e3:8.1f} us "
          f"{flops / cublas / 1e9:7.1f} TF | ratio {cublas / ours:.2f}", flush=True)


def run_gemm(dev, small: bool) -> None:
    if small:
        gemm_case(dev, "square", 16384, 4096, 4096)
        return
    rows = 32768
    print(f"resident CTA pairs: {native.lib().ajb_gemm_pair_capacity()} (AJB_GEMM_PAIR=0 keeps every product on the "
          f"single-CTA kernel)", flush=True)
    gemm_case(dev, "fwd qkv", rows, 4096, 2048)
    gemm_case(dev, "fwd w13", rows, 11264, 2048)
    gemm_case(dev, "fwd w2", rows, 2048, 5632)
    gemm_case(dev, "fwd o", rows, 2048, 2048)
    gemm_case(dev, "fwd head chunk", 8192, 32000, 2048)
    gemm_case(dev, "dgrad w13", rows, 2048, 11264, b_mn=True)
    gemm_case(dev, "dgrad w2", rows, 5632, 2048, b_mn=True)
    gemm_case(dev, "dgrad qkv", rows, 2048, 4096, b_mn=True)
    gemm_case(dev, "wgrad w13 (f32 add)", 11264, 2048, rows, a_mn=True, b_mn=True, epilogue=3)
    gemm_case(dev, "wgrad w2 (f32 add)", 2048, 5632, rows, a_mn=True, b_mn=True, epilogue=3)
    gemm_case(dev, "wgrad qkv (f32 add)", 4096, 2048, rows, a_mn=True, b_mn=True, epilogue=3)
    gemm_case(dev, "square 8192", 8192, 8192, 8192)


def run_flash(dev, small: bool, head_dim: int = 128) -> None:
    B, T, Hq, Hkv = (2 if small else 8), 4096, 16, 8
    qkv = (torch.randn(B, T, (Hq + 2 * Hkv) * head_dim, device=dev) * 0.5).to(torch.bfloat16)
    out = torch.empty(B, T, Hq * head_dim, device=dev, dtype=torch.bfloat16)
    lse = torch.empty(B, Hq, T, device=dev)
    scale, width = 1 / math.sqrt(head_dim), qkv.shape[-1]
    stream = native.stream_ptr
    fwd = lambda: native.call("ajb_flash_fwd", qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, Hq, Hkv, head_dim,
                              width, 1, scale, stream())
    t = timeit(fwd)
    flops = 4 * B * Hq * T * T * head_dim / 2
    print(f"flash fwd  B{B} T{T} H{Hq}/{Hkv} d{head_dim}: {t * 1e3:8.1f} us {flops / t / 1e9:7.1f} TF", flush=True)
    dout, delta, dqkv = torch.randn_like(out), torch.empty_like(lse), torch.empty_like(qkv)
    acc = torch.empty(B * Hq * (-(-T // 64) * 64) * head_dim, device=dev)
    for label, acc_ptr in (("fused", acc.data_ptr()), ("two-kernel", None)):
        bwd = lambda: native.call("ajb_flash_bwd", qkv.data_ptr(), out.data_ptr(), dout.data_ptr(), lse.data_ptr(),
                                  delta.data_ptr(), dqkv.data_ptr(), acc_ptr, B, T, Hq, Hkv, head_dim, width, 1, scale, stream())
        t = timeit(bwd)
        print(f"flash bwd ({label:10s}): {t * 1e3:8.1f} us {2.5 * flops / t / 1e9:7.1f} TF (five-product accounting)", flush=True)


def run_norm(dev, small: bool) -> None:
    rows, dim = (8192 if small else 32768), 2048
    x = torch.randn(rows, dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    delta = torch.randn_like(x)
    gain = torch.ones(dim, device=dev, dtype=torch.bfloat16, requires_grad=True)
    h, y = ops.add_rms_norm(x, delta, gain)
    gy = torch.randn_like(y)
    nbytes = 4 * rows * dim * 2
    t = timeit(lambda: ops.add_rms_norm(x.detach(), delta, gain.detach()))
    print(f"add + rmsnorm fwd [{rows} x {dim}]: {t * 1e3:8.1f} us {nbytes / t / 1e6:7.0f} GB/s", flush=True)
    t = timeit(lambda: torch.autograd.grad([h, y], [x], [gy, gy], retain_graph=True))
    print(f"add + rmsnorm bwd [{rows} x {dim}]: {t * 1e3:8.1f} us {nbytes / t / 1e6:7.0f} GB/s", flush=True)


def run_decode_gemm(dev, small: bool) -> None:
    """Decoding GEMMs of the 8B block: few activation rows, weights streamed once per call (L2 flushed in between by a
    256 MB memset whose own time is subtracted); bytes = the weight matrix."""
    shapes = ((6144, 4096),) if small else ((6144, 4096), (4096, 4096), (28672, 4096), (4096, 14336), (128256, 4096))
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    base = timeit(lambda: flush.zero_(), iters=20)
    with torch.no_grad():
        for rows in ((64,) if small else (16, 64, 128, 256)):
            for n, k in shapes:
                x = torch.randn(rows, k, device=dev).to(torch.bfloat16)
                w = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)

                def ours():
                    flush.zero_()
                    ops.linear(x, w)

                def library():
                    flush.zero_()
                    torch.matmul(x, w.t())

                t_ours, t_lib = timeit(ours, iters=20) - base, timeit(library, iters=20) - base
                gb = n * k * 2 / 1e6
                print(f"decode rows {rows:3d} w [{n} x {k}]: ours {t_ours * 1e3:7.1f} us {gb / t_ours:6.0f} GB/s | "
                      f"cuBLAS {t_lib * 1e3:7.1f} us {gb / t_lib:6.0f} GB/s", flush=True)
                del w


def run_paged(dev, small: bool) -> None:
    """Decode attention over a paged cache: bytes = K and V of every cached token, once. Few sequences with long contexts
    are where cutting a sequence over several CTAs matters; many sequences fill the device on their own."""
    from ajllm_b200.engine.kv_cache import PagedKVCache
    from ajllm_b200.ops import serving

    heads, kv_heads, hd = 32, 8, 128
    cases = ((16, 2048),) if small else ((16, 1024), (16, 4096), (64, 2048), (256, 1280))
    for seqs, ctx in cases:
        blocks_per = (ctx + 15) // 16
        cache = PagedKVCache(1, seqs * blocks_per + 1, 16, kv_heads, hd, torch.bfloat16, dev)
        cache.keys[0].normal_(0, 0.5)
        cache.values[0].normal_(0, 0.5)
        tables = torch.arange(seqs * blocks_per, dtype=torch.int32, device=dev).view(seqs, blocks_per)
        q = (torch.randn(seqs, heads, hd, device=dev) * 0.5).to(torch.bfloat16)
        plan = serving.PagedPlan(tables, [1] * seqs, [ctx] * seqs, heads, kv_heads)
        nbytes = 2 * seqs * ctx * kv_heads * hd * 2
        line = f"paged decode {seqs:3d} seqs x {ctx:4d} keys:"
        for label, forced in (("one CTA per (seq, kv head)", 1), ("split", None)):
            original = serving.paged_splits
            if forced is not None:
                serving.paged_splits = lambda ctas, max_context: 1
            try:
                t = timeit(lambda: serving.paged_attention_planned(q, cache.keys[0], cache.values[0], plan), iters=20)
                parts = serving.paged_splits(seqs * kv_heads, ctx)
            finally:
                serving.paged_splits = original
            line += f"  {label} ({parts} part{'s' if parts > 1 else ''}) {t * 1e3:6.1f} us {nbytes / t / 1e6:6.0f} GB/s |"
        print(line, flush=True)


def run_sampler(dev, small: bool) -> None:
    from ajllm_b200.ops import serving

    vocab = 128256
    for rows in ((16,) if small else (16, 64, 256)):
        logits = torch.randn(rows, vocab, device=dev)
        zeros = torch.zeros(rows, device=dev)
        ones = torch.ones(rows, device=dev)
        seeds = torch.arange(rows, dtype=torch.int64, device=dev)
        counters = torch.zeros(rows, dtype=torch.int64, device=dev)
        greedy = timeit(lambda: serving.sample_rows(logits, zeros, ones, seeds, counters), iters=20)
        sampled = timeit(lambda: serving.sample_rows(logits, ones, ones, seeds, counters), iters=20)
        nbytes = rows * vocab * 4
        print(f"sampler {rows:3d} rows x {vocab}: greedy {greedy * 1e3:6.1f} us ({nbytes / greedy / 1e6:5.0f} GB/s) | "
              f"temperature 1 {sampled * 1e3:6.1f} us", flush=True)


def run_fp8(dev, small: bool) -> None:
    """Block-scaled fp8 GEMM (128 x 128 weight blocks, per-token activation scales) against the bf16 GEMM of the same shape."""
    from ajllm_b200.engine.quant import Fp8Weight, fp8_linear

    shapes = ((4096, 4096, 4096),) if small else ((64, 6144, 4096), (64, 28672, 4096), (4096, 6144, 4096), (8192, 28672, 4096))
    with torch.no_grad():
        for m, n, k in shapes:
            x = torch.randn(m, k, device=dev).to(torch.bfloat16)
            w = (torch.randn(n, k, device=dev) * 0.02).to(torch.bfloat16)
            q = Fp8Weight.from_dense(w)
            t8 = timeit(lambda: fp8_linear(x, q))
            t16 = timeit(lambda: ops.linear(x, w))
            flops = 2 * m * n * k
            print(f"fp8 block-scaled m{m} n{n} k{k}: fp8 {t8 * 1e3:8.1f} us {flops / t8 / 1e9:7.1f} TF | bf16 {t16 * 1e3:8.1f} us "
                  f"{flops / t16 / 1e9:7.1f} TF", flush=True)


def run_grad_reduce(dev, small: bool) -> None:
    """The gradient reduce-scatter kernel as rank 0 of a group whose peers' buffers are tensors on this device and whose
    handshake words are preset (nothing crosses NVLink: this is the kernel's own cost at HBM speed)."""
    import ctypes

    from ajllm_b200.parallel.grad_reduce import FusedGradReduce, _Args
    fn = native.lib().ajb_grad_reduce_scatter
    fn.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p]
    fn.restype = ctypes.c_int
    for world in ((2,) if small else (2, 8)):
        shard = (8 if small else 32) * 1024 * 1024
        buffers = [torch.randn(world * shard, device=dev) for _ in range(world)]
        flags = torch.zeros(32, dtype=torch.int32, device=dev)
        counter = torch.zeros(4, dtype=torch.int32, device=dev)
        dst = torch.zeros(shard, device=dev)
        partials = torch.zeros(FusedGradReduce.CTAS, device=dev)
        epoch = [0]

        def launch():
            epoch[0] += 1
            flags[:16] = epoch[0]          # every peer's "ready" and "done" word for this call
            a = _Args()
            a.world, a.rank, a.shard_elems = world, 0, shard
            for r in range(world):
                a.full_ptrs[r] = buffers[r].data_ptr()
                a.ready_ptrs[r] = flags.data_ptr()
                a.done_ptrs[r] = flags.data_ptr() + 8 * 4
            a.dst, a.accumulate, a.scale = dst.data_ptr(), 1, 1.0
            a.sumsq_partials, a.ctas = partials.data_ptr(), FusedGradReduce.CTAS
            a.epoch, a.local_counter = epoch[0], counter.data_ptr()
            assert fn(ctypes.byref(a), native.stream_ptr()) == 0

        t = timeit(launch, iters=10)
        nbytes = (world + 2) * shard * 4        # world slices read, the shard read and written
        print(f"grad reduce-scatter as rank 0 of {world}: shard {shard * 4 / 2**20:.0f} MiB, {t * 1e3:7.1f} us "
              f"{nbytes / t / 1e6:6.0f} GB/s", flush=True)
    print("kernel status", native.check_status(False))


def run_moe_exchange(dev, small: bool) -> None:
    """Expert dispatch (push) and combine (pull) as rank 0 of an 8-rank group whose peers' buffers are tensors on this
    device and whose handshake words are preset: the kernels' own cost at HBM speed, nothing crosses NVLink."""
    import ctypes

    from ajllm_b200.parallel.moe_exchange import _Args
    lib = native.lib()
    push, pull = lib.ajb_moe_push_rows, lib.ajb_moe_pull_rows
    push.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    pull.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    push.restype = pull.restype = ctypes.c_int
    ep, local_experts, top_k, dim = 8, 8, 6, 2048
    tokens = 4096 if small else 16384
    experts = ep * local_experts
    capacity = int(1.25 * tokens * top_k / experts)
    stride = (capacity + 127) // 128 * 128
    choice = torch.rand(tokens, experts, device=dev).topk(top_k, dim=1).indices
    # position of each assignment inside its expert = its rank among the assignments to that expert
    flat = choice.reshape(-1)
    order = torch.argsort(flat, stable=True)
    ranks = torch.empty_like(order)
    counts = torch.bincount(flat, minlength=experts)
    starts = torch.cumsum(counts, 0) - counts
    ranks[order] = torch.arange(flat.numel(), device=dev) - starts[flat[order]]
    slots = torch.where(ranks < capacity, flat * stride + ranks, torch.full_like(flat, -1)).view(tokens, top_k).to(torch.int32)
    rows = torch.randn(tokens, dim, device=dev).to(torch.bfloat16)
    gates = torch.rand(tokens, top_k, device=dev)
    buffers = [torch.zeros(local_experts * ep * stride, dim, device=dev, dtype=torch.bfloat16) for _ in range(ep)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(ep)]
    counts_sym = [torch.zeros(4096, dtype=torch.int32, device=dev) for _ in range(ep)]
    kept = counts.clamp(max=capacity).to(torch.int32)
    local = torch.zeros(4, dtype=torch.int32, device=dev)
    out = torch.empty(tokens, dim, device=dev, dtype=torch.bfloat16)
    epoch = [0]

    def args():
        epoch[0] += 1
        flags[0][:24] = epoch[0]            # arrival, release and ready words of every peer for this call
        a = _Args()
        a.tokens, a.top_k, a.dim, a.ep, a.rank = tokens, top_k, dim, ep, 0
        a.local_experts, a.stride = local_experts, stride
        a.slots = slots.data_ptr()
        for r in range(ep):
            a.peer_buffers[r] = buffers[r].data_ptr()
            a.flag_ptrs[r] = flags[r].data_ptr()
            a.peer_counts[r] = counts_sym[r].data_ptr()
        a.counts = kept.data_ptr()
        a.epoch, a.local_counter = epoch[0], local.data_ptr()
        return a

    def do_push():
        a = args()
        assert push(ctypes.byref(a), rows.data_ptr(), None, native.stream_ptr()) == 0

    def do_pull():
        a = args()
        assert pull(ctypes.byref(a), out.data_ptr(), gates.data_ptr(), None, None, native.stream_ptr()) == 0

    moved = int((slots >= 0).sum()) * dim * 2
    t_push, t_pull = timeit(do_push), timeit(do_pull)
    print(f"expert dispatch as rank 0 of {ep}: {tokens} tokens x top-{top_k}, {moved / 1e6:.0f} MB of rows: push {t_push * 1e3:7.1f} us "
          f"({2 * moved / t_push / 1e6:5.0f} GB/s read + written) | pull + weighted sum {t_pull * 1e3:7.1f} us "
          f"({moved / t_pull / 1e6:5.0f} GB/s read)", flush=True)
    print("kernel status", native.check_status(False))


def run_swiglu(dev, small: bool) -> None:
    """The SwiGLU block's first projection with the activation in its epilogue, and the gradient of the pairs from the
    epilogue of d_out @ W2, each against the plain GEMM followed by the pointwise kernel."""
    from ajllm_b200.ops import functional
    rows, d_model, d_ff = (8192, 2048, 2816) if small else (32768, 2048, 5632)
    bf = torch.bfloat16
    x = torch.randn(rows, d_model, device=dev, dtype=bf)
    w13 = (torch.randn(2 * d_ff, d_model, device=dev) * d_model ** -0.5).to(bf)
    w2 = (torch.randn(d_model, d_ff, device=dev) * d_ff ** -0.5).to(bf)
    d_out = torch.randn(rows, d_model, device=dev, dtype=bf)
    gate_up = torch.empty(rows, 2 * d_ff, device=dev, dtype=bf)
    act = torch.empty(rows, d_ff, device=dev, dtype=bf)
    d_act = torch.empty(rows, d_ff, device=dev, dtype=bf)
    d_gate_up = torch.empty(rows, 2 * d_ff, device=dev, dtype=bf)
    stream = native.stream_ptr

    def fwd_fused():
        functional._gemm_swiglu(x, w13, gate_up, act, rows, 2 * d_ff, d_model, backward=False)

    def fwd_fused_act_only():
        functional._gemm_swiglu(x, w13, None, act, rows, 2 * d_ff, d_model, backward=False)

    def fwd_gemm():
        ops.gemm(x, w13, gate_up, rows, 2 * d_ff, d_model)

    def fwd_pointwise():
        native.call("ajb_swiglu_fwd", gate_up.data_ptr(), act.data_ptr(), rows, d_ff, stream())

    def bwd_fused():
        functional._gemm_swiglu(d_out, w2, gate_up, d_gate_up, rows, d_ff, d_model, backward=True)

    def bwd_gemm():
        ops.gemm(d_out, w2, d_act, rows, d_ff, d_model, b_mn_major=True)

    def bwd_pointwise():
        native.call("ajb_swiglu_bwd", gate_up.data_ptr(), d_act.data_ptr(), d_gate_up.data_ptr(), rows, d_ff, stream())

    fwd_gemm()
    t = {name: timeit(fn) * 1e3 for name, fn in [("fwd_fused", fwd_fused), ("fwd_act_only", fwd_fused_act_only),
                                                 ("fwd_gemm", fwd_gemm), ("fwd_pointwise", fwd_pointwise),
                                                 ("bwd_fused", bwd_fused), ("bwd_gemm", bwd_gemm), ("bwd_pointwise", bwd_pointwise)]}
    print(f"SwiGLU block, {rows} rows, d_model {d_model}, d_ff {d_ff}:", flush=True)
    print(f"  forward  x W13^T + activation: one kernel {t['fwd_fused']:7.1f} us (activation only, inference: {t['fwd_act_only']:7.1f} us) | "
          f"GEMM {t['fwd_gemm']:7.1f} + pointwise {t['fwd_pointwise']:6.1f} = {t['fwd_gemm'] + t['fwd_pointwise']:7.1f} us", flush=True)
    print(f"  backward d_out W2 -> d(gate, up): one kernel {t['bwd_fused']:7.1f} us | "
          f"GEMM {t['bwd_gemm']:7.1f} + pointwise {t['bwd_pointwise']:6.1f} = {t['bwd_gemm'] + t['bwd_pointwise']:7.1f} us", flush=True)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", default="all", choices=["all", "gemm", "decode", "flash", "flash64", "norm", "paged", "sampler",
                                                      "fp8", "grad_reduce", "moe_exchange", "swiglu"])
    ap.add_argument("--small", action="store_true", help="one small shape per case (a few hundred MB on the device)")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("bench_kernels.py needs a GPU")
    dev = torch.device("cuda")
    torch.manual_seed(0)
    if args.case in ("all", "gemm"):
        run_gemm(dev, args.small)
    if args.case in ("all", "decode"):
        run_decode_gemm(dev, args.small)
    if args.case in ("all", "flash"):
        run_flash(dev, args.small)
    if args.case in ("all", "flash64"):
        run_flash(dev, args.small, head_dim=64)
    if args.case in ("all", "norm"):
        run_norm(dev, args.small)
    if args.case in ("all", "paged"):
        run_paged(dev, args.small)
    if args.case in ("all", "sampler"):
        run_sampler(dev, args.small)
    if args.case in ("all", "fp8"):
        run_fp8(dev, args.small)
    if args.case in ("all", "grad_reduce"):
        run_grad_reduce(dev, args.small)
    if args.case in ("all", "moe_exchange"):
        run_moe_exchange(dev, args.small)
    if args.case in ("all", "swiglu"):
        run_swiglu(dev, args.small)
    print("kernel status", native.lib().ajb_check_status())


if __name__ == "__main__":
    main()
