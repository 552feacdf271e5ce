"""Expert-parallel token exchange over symmetric NVLink memory.

Dispatch writes every kept (token, choice) row straight into the owning rank's expert-major buffer and
combine reads each token's expert outputs back from the ranks that computed them, both from inside one
kernel each (``csrc/moe.cu``: peer stores / peer loads plus flag handshakes), replacing the two
``all_to_all`` collectives and the index gathers/scatters around them. The per-(expert, source) row
counts travel with the dispatch so the batched expert GEMMs skip padding. Backward passes reuse the same
two kernels with the roles swapped (dispatch^T = pull, combine^T = scaled push + dot products for the
gate gradients). The NCCL ``all_to_all_single`` path in :mod:`ajllm_b200.models.moe` is the baseline.
"""

from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ajllm_b200.ops import native
from ajllm_b200.utils.timing import nvtx_range


class _Args(ctypes.Structure):
    _fields_ = [
        ("tokens", ctypes.c_int), ("top_k", ctypes.c_int), ("dim", ctypes.c_int), ("ep", ctypes.c_int),
        ("rank", ctypes.c_int), ("local_experts", ctypes.c_int), ("stride", ctypes.c_int), ("pad", ctypes.c_int),
        ("slots", ctypes.c_void_p),
        ("peer_buffers", ctypes.c_void_p * 8), ("flag_ptrs", ctypes.c_void_p * 8), ("peer_counts", ctypes.c_void_p * 8),
        ("counts", ctypes.c_void_p), ("epoch", ctypes.c_uint), ("pad2", ctypes.c_uint), ("local_counter", ctypes.c_void_p),
    ]


class FusedExpertExchange:
    GUARD_ELEMENTS, GUARD_VALUE = 2048, -12345.0      # behind every symmetric row buffer (peers store with raw pointers)

    def __init__(self, group, device: torch.device) -> None:
        import torch.distributed._symmetric_memory as symm_mem

        self._symm = symm_mem
        self.group, self.device = group, device
        self.size, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.epoch = 0
        self._buffers: dict[str, tuple[torch.Tensor, list[int]]] = {}
        self._flags = symm_mem.empty(64, dtype=torch.int32, device=device)
        self._flags.zero_()
        self._flag_ptrs = list(symm_mem.rendezvous(self._flags, group).buffer_ptrs)
        self._counts = symm_mem.empty(4096, dtype=torch.int32, device=device)
        self._counts.zero_()
        self._count_ptrs = list(symm_mem.rendezvous(self._counts, group).buffer_ptrs)
        self._local = torch.zeros(4, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)
        lib = native.lib()
        self._push = lib.ajb_moe_push_rows
        self._push.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
        self._push.restype = ctypes.c_int
        self._pull = lib.ajb_moe_pull_rows
        self._pull.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p,
                               ctypes.c_void_p]
        self._pull.restype = ctypes.c_int

    def buffer(self, name: str, rows: int, dim: int) -> tuple[torch.Tensor, list[int]]:
        """Symmetric bf16 ``[rows, dim]`` buffer (allocated collectively on first use, zero-filled)."""
        need = rows * dim
        have = self._buffers.get(name)
        if have is None or have[0].numel() - self.GUARD_ELEMENTS < need:
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            buf = self._symm.empty(need + self.GUARD_ELEMENTS, dtype=torch.bfloat16, device=self.device)
            buf.zero_()
            buf[need:].fill_(self.GUARD_VALUE)
            ptrs = list(self._symm.rendezvous(buf, self.group).buffer_ptrs)
            torch.cuda.synchronize(self.device)
            dist.barrier(self.group)
            have = (buf, ptrs)
            self._buffers[name] = have
        return have[0][:need].view(rows, dim), have[1]

    def guards_intact(self) -> bool:
        """True while no peer has stored past the end of a row buffer (checked by the multi-GPU tests)."""
        return all(bool((buf[-self.GUARD_ELEMENTS:] == self.GUARD_VALUE).all()) for buf, _ in self._buffers.values())

    def _args(self, slots: torch.Tensor, dim: int, local_experts: int, stride: int, peer_ptrs: list[int],
              counts: torch.Tensor | None) -> _Args:
        self.epoch += 1
        a = _Args()
        a.tokens, a.top_k, a.dim = slots.shape[0], slots.shape[1], dim
        a.ep, a.rank, a.local_experts, a.stride = self.size, self.rank, local_experts, stride
        a.slots = slots.data_ptr()
        for r in range(self.size):
            a.peer_buffers[r] = peer_ptrs[r]
            a.flag_ptrs[r] = self._flag_ptrs[r]
            a.peer_counts[r] = self._count_ptrs[r]
        a.counts = counts.data_ptr() if counts is not None else None
        a.epoch = self.epoch & 0xFFFFFFFF
        a.local_counter = self._local.data_ptr()
        return a

    def push(self, rows: torch.Tensor, scale: torch.Tensor | None, slots: torch.Tensor, local_experts: int, stride: int,
             name: str, counts: torch.Tensor | None = None) -> torch.Tensor:
        """Send rows to their slots; returns this rank's received ``[local_experts, ep * stride, dim]`` (a copy;
        the symmetric buffer is zeroed again for its next use)."""
        dim = rows.shape[1]
        total = local_experts * self.size * stride
        buf, ptrs = self.buffer(name, total, dim)
        args = self._args(slots, dim, local_experts, stride, ptrs, counts)
        native.launch_count += 1
        with nvtx_range("moe_dispatch"):
            status = self._push(ctypes.byref(args), rows.data_ptr(), native.ptr(scale), native.stream_ptr())
        if status != 0:
            raise RuntimeError(f"ajb_moe_push_rows failed: {native.lib().ajb_last_error().decode()}")
        received = buf.clone().view(local_experts, self.size * stride, dim)
        buf.zero_()
        return received

    def received_counts(self, local_experts: int) -> torch.Tensor:
        return self._counts[: local_experts * self.size].clone().view(local_experts, self.size)

    def pull(self, source: torch.Tensor, slots: torch.Tensor, weights: torch.Tensor | None, local_experts: int,
             stride: int, name: str, upstream: torch.Tensor | None = None, want_rows: bool = True):
        """Stage ``source [local_experts, ep * stride, dim]`` in the symmetric buffer and gather: returns
        ``(rows [tokens, dim] or None, dots [tokens, top_k] or None)``."""
        dim = source.shape[-1]
        total = local_experts * self.size * stride
        buf, ptrs = self.buffer(name, total, dim)
        buf.copy_(source.reshape(total, dim))
        args = self._args(slots, dim, local_experts, stride, ptrs, None)
        out = torch.empty(slots.shape[0], dim, dtype=torch.bfloat16, device=self.device) if want_rows else None
        dots = torch.zeros(slots.shape, dtype=torch.float32, device=self.device) if upstream is not None else None
        native.launch_count += 1
        with nvtx_range("moe_combine"):
            status = self._pull(ctypes.byref(args), native.ptr(out), native.ptr(weights), native.ptr(upstream), native.ptr(dots),
                                native.stream_ptr())
        if status != 0:
            raise RuntimeError(f"ajb_moe_pull_rows failed: {native.lib().ajb_last_error().decode()}")
        return out, dots


class _DispatchFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, flat, slots, counts, exchange: FusedExpertExchange, local_experts: int, stride: int):
        grouped = exchange.push(flat.contiguous(), None, slots, local_experts, stride, "x", counts)
        ctx.exchange, ctx.meta = exchange, (local_experts, stride)
        ctx.save_for_backward(slots)
        return grouped

    @staticmethod
    def backward(ctx, grad_grouped):
        (slots,) = ctx.saved_tensors
        local_experts, stride = ctx.meta
        grad_flat, _ = ctx.exchange.pull(grad_grouped.contiguous(), slots, None, local_experts, stride, "gx")
        return grad_flat, None, None, None, None, None


class _CombineFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, expert_out, gates, slots, exchange: FusedExpertExchange, local_experts: int, stride: int):
        out, _ = exchange.pull(expert_out, slots, gates, local_experts, stride, "y")
        ctx.exchange, ctx.meta = exchange, (local_experts, stride)
        ctx.save_for_backward(expert_out, gates, slots)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        expert_out, gates, slots = ctx.saved_tensors
        local_experts, stride = ctx.meta
        grad_out = grad_out.contiguous()
        # gate gradients: dot of the upstream gradient with each selected expert output row
        _, dots = ctx.exchange.pull(expert_out, slots, None, local_experts, stride, "y", upstream=grad_out, want_rows=False)
        # gradient of the expert outputs: the token's upstream gradient, scaled by its gate, sent to the slot
        grad_expert = ctx.exchange.push(grad_out, gates, slots, local_experts, stride, "gy")
        return grad_expert, dots, None, None, None, None


def dispatch(flat, slots, counts, exchange, local_experts, stride):
    return _DispatchFn.apply(flat, slots, counts, exchange, local_experts, stride)


def combine(expert_out, gates, slots, exchange, local_experts, stride):
    return _CombineFn.apply(expert_out, gates, slots, exchange, local_experts, stride)
