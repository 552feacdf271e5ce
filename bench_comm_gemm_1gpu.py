"""The fused tensor-parallel GEMM kernels (csrc/comm_gemm.cu) on ONE GPU, as rank 0 of a 2-rank group whose
"peer" buffers are ordinary tensors on the same device and whose handshake words are preset by the host.

This exists for profiler captures (a profiler must not wrap a multi-rank job) and as a single-GPU numerics check
of the four modes; nothing crosses NVLink here, so the timings say what the kernel costs when the transfer is
free, not how well it hides a real one (that is `bench.py --gpus N` and tests/test_gpu_fused_tp.py).

    python bench_comm_gemm_1gpu.py            # all modes, check + time
    python bench_comm_gemm_1gpu.py --small    # smaller shapes for a profiler capture
    python bench_comm_gemm_1gpu.py --tp 8     # rank 0 of an 8-rank group: shard order, per-shard arrival groups and
                                              # per-destination credits of the all-gather and reduce-scatter modes
"""

from __future__ import annotations

import argparse

import torch

from ajllm_b200.ops import native
from ajllm_b200.parallel.emulated_group import (MODE_ALL_GATHER, MODE_ALL_REDUCE, MODE_GATHER_WEIGHT,
                                                MODE_REDUCE_SCATTER, EmulatedGroup)

TP = 2          # --tp 4 / 8 emulate rank 0 of a larger group (all-gather and reduce-scatter modes)


def timeit(fn, iters=5, warmup=2):
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


def rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm())


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--small", action="store_true")
    ap.add_argument("--tp", type=int, default=2, choices=[2, 4, 8], help="size of the emulated group (rank 0 runs)")
    args = ap.parse_args()
    global TP
    TP = args.tp
    dev = torch.device("cuda")
    torch.manual_seed(0)
    em = EmulatedGroup(dev, TP)
    m, n, k = (8192, 2048, 2048) if args.small else (16384, 4096, 4096)
    m_local = m // TP
    bf = torch.bfloat16
    x = (torch.randn(m, k, device=dev) * 0.5).to(bf)
    w = (torch.randn(n, k, device=dev) * 0.05).to(bf)
    flops = 2 * m * n * k

    # all-gather -> GEMM: rank 0 owns rows [0, m_local), the "peer" staging buffer holds the other half
    stage = [x[r * m_local:(r + 1) * m_local].contiguous() for r in range(TP)]
    gathered = torch.zeros(m, k, device=dev, dtype=bf)
    gathered[:m_local].copy_(stage[0])
    out = torch.empty(m, n, device=dev, dtype=bf)
    run = lambda: em.launch(MODE_ALL_GATHER, m, n, k, out, b=w, gathered=gathered, stage=stage)
    t = timeit(run)
    print(f"all-gather -> GEMM   m{m} n{n} k{k}: {t * 1e3:8.1f} us {flops / t / 1e9:7.1f} TF  rel.err {rel(out, x.float() @ w.float().t()):.1e}", flush=True)
    assert torch.equal(gathered, x), "every shard of the gathered activations must be in place after the kernel"

    # GEMM -> reduce-scatter: rank 0 multiplies its K slice; the peer's partial for rank 0's rows is placed by the host
    x1 = (torch.randn(m, k, device=dev) * 0.5).to(bf)       # the peer's activations (its K slice)
    w1 = (torch.randn(n, k, device=dev) * 0.05).to(bf)
    recv = [torch.zeros(TP, m_local, n, device=dev, dtype=bf) for _ in range(TP)]
    peer_partial = x1[:m_local].float() @ w1.float().t()
    for r in range(1, TP):
        recv[0][r].copy_((peer_partial * (0.5 + 0.25 * r)).to(bf))
    out_rs = torch.empty(m_local, n, device=dev, dtype=bf)
    tiles = (m_local // 128) * ((n + 255) // 256)
    run = lambda: em.launch(MODE_REDUCE_SCATTER, m, n, k, out_rs, b=w, a=x, recv=recv, tiles_for_count=tiles)
    t = timeit(run)
    want = x[:m_local].float() @ w.float().t() + sum(recv[0][r].float() for r in range(1, TP))
    print(f"GEMM -> reduce-scatter m{m} n{n} k{k}: {t * 1e3:8.1f} us {flops / t / 1e9:7.1f} TF  rel.err {rel(out_rs, want):.1e}", flush=True)

    if TP != 2:      # the two remaining modes are emulated for a group of two only
        print("kernel status", native.lib().ajb_check_status())
        return

    # GEMM -> all-reduce (decoding rows)
    rows = 128
    xa = x[:rows].contiguous()
    recv_ar = [torch.zeros(TP, rows, n, device=dev, dtype=bf) for _ in range(TP)]
    recv_ar[0][1].copy_((x1[:rows].float() @ w1.float().t()).to(bf))
    out_ar = torch.empty(rows, n, device=dev, dtype=bf)
    tiles = (rows // 128) * ((n + 255) // 256)
    run = lambda: em.launch(MODE_ALL_REDUCE, rows, n, k, out_ar, b=w, a=xa, recv=recv_ar, tiles_for_count=tiles, a_rows=rows)
    t = timeit(run)
    want = xa.float() @ w.float().t() + recv_ar[0][1].float()
    print(f"GEMM -> all-reduce    rows{rows} n{n} k{k}: {t * 1e3:8.1f} us                rel.err {rel(out_ar, want):.1e}", flush=True)

    # gather-weight GEMM: W sits at an offset inside a flat buffer cut into two slices
    offset = 4096
    shard = (offset + n * k + 4096 + 15) // 16 * 8
    flat_all = torch.zeros(TP * shard, device=dev, dtype=bf)
    flat_all[offset:offset + n * k].copy_(w.reshape(-1))
    stage_w = [flat_all[:shard].contiguous(), flat_all[shard:].contiguous()]
    flat = torch.zeros(TP * shard, device=dev, dtype=bf)
    flat[:shard].copy_(stage_w[0])
    out_gw = torch.empty(m, n, device=dev, dtype=bf)
    run = lambda: em.launch(MODE_GATHER_WEIGHT, m, n, k, out_gw, b=flat, a=x, gathered=flat, stage=stage_w,
                            shard_elems=shard, b_offset=offset)
    t = timeit(run)
    print(f"gather-weight GEMM   m{m} n{n} k{k}: {t * 1e3:8.1f} us {flops / t / 1e9:7.1f} TF  rel.err {rel(out_gw, x.float() @ w.float().t()):.1e}", flush=True)
    print("kernel status", native.lib().ajb_check_status())


if __name__ == "__main__":
    main()
