"""Kernel microbenchmarks on one B200: the tcgen05 GEMM against cuBLAS on the layer shapes of the flagship
model, the attention kernels, the fused norm kernels, and the tensor-pipe probe.

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
        for rows in ((64,) if small else (16, 64, 128)):
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


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--case", default="all", choices=["all", "gemm", "decode", "flash", "flash64", "norm"])
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
    print("kernel status", native.lib().ajb_check_status())


if __name__ == "__main__":
    main()
