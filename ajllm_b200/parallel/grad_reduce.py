"""Gradient reduce-scatter over symmetric NVLink memory, fused with shard accumulation and sum of squares.

The sharded data-parallel wrapper lets the weight-gradient GEMMs of a unit accumulate into one fp32
buffer per rank. When that buffer lives in symmetric memory, ``csrc/grad_reduce.cu`` replaces the NCCL
``reduce_scatter`` + ``add_`` + (at the optimizer step) the separate sum-of-squares pass: every rank pulls
its slice of each peer's buffer, adds the slices in rank order, accumulates into its gradient shard and
leaves per-CTA partial sums of squares of the updated shard. The reference reduces with
``dist.reduce_scatter_tensor`` and clips in eager code (``ajllm/training/distributed.py:107-124``,
``ajllm/training/trainer.py:30-40``).
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ajllm_b200.ops import native
from ajllm_b200.utils.timing import nvtx_range

_MAX_RANKS = 8


class _Args(ctypes.Structure):
    _fields_ = [
        ("world", ctypes.c_int), ("rank", ctypes.c_int), ("shard_elems", ctypes.c_longlong),
        ("full_ptrs", ctypes.c_void_p * _MAX_RANKS), ("dst", ctypes.c_void_p),
        ("accumulate", ctypes.c_int), ("scale", ctypes.c_float), ("sumsq_partials", ctypes.c_void_p),
        ("ctas", ctypes.c_int),
        ("ready_ptrs", ctypes.c_void_p * _MAX_RANKS), ("done_ptrs", ctypes.c_void_p * _MAX_RANKS),
        ("epoch", ctypes.c_uint), ("local_counter", ctypes.c_void_p),
    ]


class FusedGradReduce:
    """Owns the symmetric full-gradient buffer of ``elements`` floats and the handshake words."""

    CTAS = 64          # enough 16-byte loads in flight to fill the NVLink ports; leaves SMs to other streams
    GUARD_FLOATS, GUARD_VALUE = 1024, -6.02e23     # behind the payload: peers address this buffer with raw pointers

    def __init__(self, group, device: torch.device, elements: int) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.device = group, device
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        if not 1 <= self.world <= _MAX_RANKS:
            raise ValueError("fused gradient reduce-scatter supports up to 8 ranks")
        self._whole = symm_mem.empty(elements + self.GUARD_FLOATS, dtype=torch.float32, device=device)
        self._whole.zero_()
        self._whole[elements:].fill_(self.GUARD_VALUE)
        self.buffer = self._whole[:elements]
        self._buffer_ptrs = list(symm_mem.rendezvous(self._whole, group).buffer_ptrs)
        self._flags = symm_mem.empty(32, dtype=torch.int32, device=device)     # [0:8] ready, [8:16] done
        self._flags.zero_()
        self._flag_ptrs = list(symm_mem.rendezvous(self._flags, group).buffer_ptrs)
        self._counter = torch.zeros(4, dtype=torch.int32, device=device)
        self.epoch = 0
        torch.cuda.synchronize(device)
        dist.barrier(group)
        fn = native.lib().ajb_grad_reduce_scatter
        fn.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p]
        fn.restype = ctypes.c_int
        self._fn = fn

    def guards_intact(self) -> bool:
        """True while nothing (a weight-gradient epilogue, a peer's kernel) has written behind the end of the buffer."""
        return bool((self._whole[self.buffer.numel():] == self.GUARD_VALUE).all())

    def reduce_into(self, dst: torch.Tensor, shard_elems: int, accumulate: bool = True, scale: float = 1.0,
                    sumsq_partials: torch.Tensor | None = None) -> None:
        """``dst (+)= scale * sum_r buffer_r[rank * shard_elems : (rank + 1) * shard_elems]``; optionally
        ``sumsq_partials[c] = sum of squares of the part of the updated dst that CTA c handled``."""
        if dst.dtype != torch.float32 or not dst.is_contiguous() or dst.numel() != shard_elems:
            raise ValueError("dst must be a contiguous fp32 tensor of shard_elems elements")
        if self.world * shard_elems > self.buffer.numel():
            raise ValueError("the symmetric gradient buffer is smaller than world * shard_elems")
        if sumsq_partials is not None and (sumsq_partials.dtype != torch.float32 or sumsq_partials.numel() < self.CTAS):
            raise ValueError(f"sumsq_partials needs {self.CTAS} fp32 slots")
        self.epoch += 1
        args = _Args()
        args.world, args.rank, args.shard_elems = self.world, self.rank, shard_elems
        for r in range(self.world):
            args.full_ptrs[r] = self._buffer_ptrs[r]
            args.ready_ptrs[r] = self._flag_ptrs[r]
            args.done_ptrs[r] = self._flag_ptrs[r] + 8 * 4
        args.dst = dst.data_ptr()
        args.accumulate, args.scale = int(accumulate), scale
        args.sumsq_partials = sumsq_partials.data_ptr() if sumsq_partials is not None else None
        args.ctas = self.CTAS
        args.epoch = self.epoch & 0xFFFFFFFF
        args.local_counter = self._counter.data_ptr()
        native.launch_count += 1
        with nvtx_range("grad_reduce_scatter"):
            status = self._fn(ctypes.byref(args), native.stream_ptr())
        if status != 0:
            raise RuntimeError(f"ajb_grad_reduce_scatter failed: {native.lib().ajb_last_error().decode()}")
