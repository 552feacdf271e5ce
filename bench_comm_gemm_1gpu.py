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
import ctypes

import torch

from ajllm_b200.ops import native
from ajllm_b200.parallel.fused import (MODE_ALL_GATHER, MODE_ALL_REDUCE, MODE_GATHER_WEIGHT, MODE_REDUCE_SCATTER,
                                       _CommArgs)

TP, RANK = 2, 0          # --tp 4 / 8 emulate rank 0 of a larger group (all-gather and reduce-scatter modes)


class Emulated:
    def __init__(self, device) -> None:
        self.device = device
        # one flag array per "rank": [0:8] ready, [8:16] done, [16:24] arrival counters
        self.flags = [torch.zeros(64, dtype=torch.int32, device=device) for _ in range(TP)]
        self.local = torch.zeros(272, dtype=torch.int32, device=device)
        self.epoch = 0
        self.expected = 0
        fn = native.lib().ajb_comm_gemm
        fn.argtypes = [ctypes.POINTER(_CommArgs), ctypes.c_void_p]
        fn.restype = ctypes.c_int
        self.fn = fn

    def launch(self, mode, m, n, k, out, b=None, b_mn=False, a=None, gathered=None, stage=None, recv=None,
               tiles_for_count=0, a_rows=0, shard_elems=0, b_offset=0):
        self.epoch += 1
        self.expected += tiles_for_count * 4
        # what the absent peers would have written into rank 0's words
        self.flags[0][1:TP] = self.epoch                 # ready[r]
        self.flags[0][8 + 1:8 + TP] = self.epoch         # done[r]
        self.flags[0][16 + 1:16 + TP] = self.expected    # arrivals from rank r
        args = _CommArgs()
        args.mode, args.m, args.n, args.k = mode, m, n, k
        args.tp, args.rank, args.b_mn_major, args.copy_ctas = TP, RANK, int(b_mn), 20
        args.ldb = b.stride(0) if (b is not None and b.dim() == 2) else k
        args.ldc = out.stride(0)
        args.a = a.data_ptr() if a is not None else None
        args.b = b.data_ptr() if b is not None else None
        args.out = out.data_ptr()
        args.gathered = gathered.data_ptr() if gathered is not None else None
        for r in range(TP):
            args.stage_ptrs[r] = stage[r].data_ptr() if stage is not None else None
            args.recv_ptrs[r] = recv[r].data_ptr() if recv is not None else None
            args.ready_ptrs[r] = self.flags[r].data_ptr()
            args.done_ptrs[r] = self.flags[r].data_ptr() + 8 * 4
            args.counter_ptrs[r] = self.flags[r].data_ptr() + 16 * 4
        args.shard_flags = self.local.data_ptr()
        args.expected_count = self.expected & 0xFFFFFFFF
        args.epoch = self.epoch & 0xFFFFFFFF
        args.a_rows, args.shard_elems, args.b_offset_elems = a_rows, shard_elems, b_offset
        status = self.fn(ctypes.byref(args), native.stream_ptr())
        if status != 0:
            raise RuntimeError(native.lib().ajb_last_error().decode())


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
    em = Emulated(dev)
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
