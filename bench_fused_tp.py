"""Per-op timing of the fused tensor-parallel kernels against NCCL + GEMM, one process per GPU.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 bench_fused_tp.py

For each projection shape of the 1.3 B flagship block (column-parallel QKV and W1/W3, row-parallel WO and W2) the
script times, with CUDA events on the launching stream and the maximum over ranks:

  * the fused kernel (`FusedTensorParallel.all_gather_gemm` / `gemm_reduce_scatter`),
  * the same result from an NCCL collective and the plain GEMM kernel,
  * the plain GEMM and the collective on their own,

and prints the roofline target of the fused kernel: the slower of FLOPs / measured sustained cuBLAS rate and
bytes over NVLink / measured peer-copy bandwidth. Operands (tens of MB each way, rotated over several buffers so
that the set exceeds L2) are synthetic.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path

import torch
import torch.distributed as dist

sys.path.insert(0, str(Path(__file__).resolve().parent))

from ajllm_b200 import ops  # noqa: E402
from ajllm_b200.ops import native  # noqa: E402
from ajllm_b200.parallel import init_distributed  # noqa: E402
from ajllm_b200.parallel.fused import FusedTensorParallel  # noqa: E402

NVLINK_GBS = 770.0          # measured peer copy, per direction
FALLBACK_TFLOPS = 1400.0    # sustained cuBLAS bf16 when no measurement file is present


def sustained_tflops() -> float:
    path = Path(__file__).resolve().parent / "MEASURED_PEAKS.json"
    if path.is_file():
        peaks = json.loads(path.read_text())
        for key in ("bf16_tflops_sustained", "bf16_tflops"):
            if key in peaks:
                return float(peaks[key])
    return FALLBACK_TFLOPS


def timeit(fn, device, iters: int, warmup: int) -> float:
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(iters):
        fn()
    end.record()
    torch.cuda.synchronize()
    t = torch.tensor([begin.elapsed_time(end) / iters], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t) * 1e3       # microseconds


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--tokens", type=int, default=32768)
    parser.add_argument("--d-model", type=int, default=2048)
    parser.add_argument("--d-ff", type=int, default=5632)
    parser.add_argument("--iters", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    args = parser.parse_args()

    rank, world, device = init_distributed("cuda")
    peak = sustained_tflops()
    m, d = args.tokens, args.d_model
    m_local = m // world
    fused = FusedTensorParallel(dist.group.WORLD, device)
    rows = []

    def report(name, t_fused, t_lib, t_gemm, t_coll, flops, link_bytes):
        target = max(flops / (peak * 1e12), link_bytes / (NVLINK_GBS * 1e9)) * 1e6
        rows.append({"op": name, "fused_us": round(t_fused, 1), "nccl_plus_gemm_us": round(t_lib, 1),
                     "gemm_us": round(t_gemm, 1), "collective_us": round(t_coll, 1),
                     "target_us": round(target, 1), "of_target": round(target / t_fused, 3)})
        if rank == 0:
            print(f"{name:34s} fused {t_fused:7.1f} us | nccl+gemm {t_lib:7.1f} (gemm {t_gemm:6.1f} + coll {t_coll:6.1f}) | "
                  f"target {target:6.1f} us -> {target / t_fused:.2f} of target", flush=True)

    for name, n_local in (("all-gather->GEMM qkv", 2 * d // world), ("all-gather->GEMM w1w3", 2 * args.d_ff // world)):
        x = torch.randn(m_local, d, device=device, dtype=torch.bfloat16)
        w = (torch.randn(n_local, d, device=device) * 0.02).to(torch.bfloat16)
        full = torch.empty(m, d, device=device, dtype=torch.bfloat16)
        out = torch.empty(m, n_local, device=device, dtype=torch.bfloat16)

        def library():
            dist.all_gather_into_tensor(full, x)
            ops.gemm(full, w, out, m, n_local, d)

        t_f = timeit(lambda: fused.all_gather_gemm(x, w, False, n_local, d), device, args.iters, args.warmup)
        t_l = timeit(library, device, args.iters, args.warmup)
        t_g = timeit(lambda: ops.gemm(full, w, out, m, n_local, d), device, args.iters, args.warmup)
        t_c = timeit(lambda: dist.all_gather_into_tensor(full, x), device, args.iters, args.warmup)
        report(f"{name} n_local={n_local}", t_f, t_l, t_g, t_c, 2.0 * m * n_local * d,
               (world - 1) * m_local * d * 2)

    for name, k_local in (("GEMM->reduce-scatter wo", d // world), ("GEMM->reduce-scatter w2", args.d_ff // world)):
        a = torch.randn(m, k_local, device=device, dtype=torch.bfloat16)
        w = (torch.randn(d, k_local, device=device) * 0.02).to(torch.bfloat16)
        partial = torch.empty(m, d, device=device, dtype=torch.bfloat16)
        out = torch.empty(m_local, d, device=device, dtype=torch.bfloat16)

        def library():
            ops.gemm(a, w, partial, m, d, k_local)
            dist.reduce_scatter_tensor(out, partial)

        t_f = timeit(lambda: fused.gemm_reduce_scatter(a, w, False, d, k_local), device, args.iters, args.warmup)
        t_l = timeit(library, device, args.iters, args.warmup)
        t_g = timeit(lambda: ops.gemm(a, w, partial, m, d, k_local), device, args.iters, args.warmup)
        t_c = timeit(lambda: dist.reduce_scatter_tensor(out, partial), device, args.iters, args.warmup)
        report(f"{name} k_local={k_local}", t_f, t_l, t_g, t_c, 2.0 * m * d * k_local,
               (world - 1) * m_local * d * 2)

    status = native.lib().ajb_check_status()
    if rank == 0:
        print(json.dumps({"world": world, "tokens": m, "d_model": d, "d_ff": args.d_ff,
                          "sustained_tflops": peak, "nvlink_gbs": NVLINK_GBS, "kernel_status": status, "rows": rows}))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
