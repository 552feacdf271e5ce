"""One GPU playing rank 0 of a tensor-parallel group, for the kernels of ``csrc/comm_gemm.cu``.

A profiler must not wrap a multi-rank job, and a test box may have a single GPU. Here the "peer" buffers are
ordinary tensors on the same device and the words that the absent peers would have written (staging buffer
ready, buffer released, partial tiles arrived) are preset by the host before every launch, so no wait ever
runs out. Nothing crosses NVLink: the numerics of every mode, the tile order, the per-shard arrival groups, the
per-destination credits and the double-buffered call protocol are exercised; how well a real transfer hides
behind the products is measured on real groups (``bench_fused_tp.py``, ``bench.py --gpus N``).
"""

from __future__ import annotations

import ctypes

import torch

from ajllm_b200.ops import native
from ajllm_b200.parallel.fused import (MODE_ALL_GATHER, MODE_ALL_REDUCE, MODE_GATHER_WEIGHT, MODE_REDUCE_SCATTER,
                                       _CommArgs)

__all__ = ["EmulatedGroup", "MODE_ALL_GATHER", "MODE_ALL_REDUCE", "MODE_GATHER_WEIGHT", "MODE_REDUCE_SCATTER"]


class EmulatedGroup:
    """Launches ``ajb_comm_gemm`` as rank 0 of ``tp`` ranks. Flag words per "rank": [0:8] ready, [8:16] released
    (gathering calls), [16:24] arrival counters, [24:32] released (reducing calls)."""

    def __init__(self, device, tp: int = 2, copy_ctas: int = 20) -> None:
        self.device, self.tp, self.copy_ctas = device, tp, copy_ctas
        self.flags = [torch.zeros(64, dtype=torch.int32, device=device) for _ in range(tp)]
        self.local = torch.zeros(272, dtype=torch.int32, device=device)
        self.reduce_state = torch.zeros(4, dtype=torch.int32, device=device)
        self.gather_calls = 0
        self.reduce_calls = 0
        self.expected = 0
        fn = native.lib().ajb_comm_gemm
        fn.argtypes = [ctypes.POINTER(_CommArgs), ctypes.c_void_p]
        fn.restype = ctypes.c_int
        self.fn = fn

    def receive_parity(self) -> int:
        """Parity (call number & 1) of the receive buffers that the NEXT reducing call sums."""
        return (self.reduce_calls + 1) & 1

    def launch(self, mode, m, n, k, out, b=None, b_mn=False, a=None, gathered=None, stage=None, recv=None,
               recv_even=None, tiles_for_count=0, a_rows=0, shard_elems=0, b_offset=0, sm_budget=None, swiglu=0, aux=None):
        tp = self.tp
        gathers = mode in (MODE_ALL_GATHER, MODE_GATHER_WEIGHT)
        if gathers:
            self.gather_calls += 1
            self.flags[0][1:tp] = self.gather_calls                 # ready[r]: the peers' staging buffers hold this call
            self.flags[0][8 + 1:8 + tp] = self.gather_calls         # the peers are done reading this rank's buffers
        else:
            self.reduce_calls += 1
            self.expected += tiles_for_count * 4
            self.flags[0][24 + 1:24 + tp] = self.reduce_calls       # the peers released their receive buffers
            self.flags[0][16 + 1:16 + tp] = self.expected           # all partial tiles of the peers have arrived
        args = _CommArgs()
        args.mode, args.m, args.n, args.k = mode, m, n, k
        args.tp, args.rank, args.b_mn_major, args.copy_ctas = tp, 0, int(b_mn), self.copy_ctas
        args.ldb = b.stride(0) if (b is not None and b.dim() == 2) else k
        args.ldc = out.stride(0)
        args.a = a.data_ptr() if a is not None else None
        args.b = b.data_ptr() if b is not None else None
        args.out = out.data_ptr()
        args.gathered = gathered.data_ptr() if gathered is not None else None
        recv_even = recv_even if recv_even is not None else recv
        for r in range(tp):
            args.stage_ptrs[r] = stage[r].data_ptr() if stage is not None else None
            args.recv_ptrs[r] = recv[r].data_ptr() if recv is not None else None
            args.recv_ptrs_even[r] = recv_even[r].data_ptr() if recv_even is not None else None
            args.ready_ptrs[r] = self.flags[r].data_ptr()
            args.done_ptrs[r] = self.flags[r].data_ptr() + (8 if gathers else 24) * 4
            args.counter_ptrs[r] = self.flags[r].data_ptr() + 16 * 4
        args.shard_flags = self.local.data_ptr()
        args.reduce_state = self.reduce_state.data_ptr()
        args.epoch = self.gather_calls & 0xFFFFFFFF
        args.a_rows, args.shard_elems, args.b_offset_elems = a_rows, shard_elems, b_offset
        args.swiglu = swiglu
        args.aux = aux.data_ptr() if aux is not None else None
        args.ld_aux = aux.stride(0) if aux is not None else 0
        native.launch_count += 1
        with native.sm_budget(sm_budget):
            status = self.fn(ctypes.byref(args), native.stream_ptr())
        if status != 0:
            raise RuntimeError(native.lib().ajb_last_error().decode())
