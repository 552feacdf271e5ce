"""Megatron-style tensor parallelism with sequence-parallel activations.

Between blocks the residual stream is sharded by token: rank ``r`` owns rows
``[r*N/tp, (r+1)*N/tp)`` of the flattened ``[N, d_model]`` activations. A column-parallel projection
(q|k|v, SwiGLU gate/up) all-gathers the rows and multiplies by this rank's slice of output features;
a row-parallel projection (attention output, SwiGLU down) multiplies by this rank's slice of input
features and reduce-scatters the partial sums back to token shards. Backward mirrors it
(all-gather <-> reduce-scatter). Embeddings, norm gains and the LM head are replicated and work on
the local tokens only; their gradients are summed over the group once per step.

``gather_linear`` / ``linear_scatter`` are the two fusion points: on CUDA with symmetric memory
available they run as single kernels that overlap the NVLink transfer with the tensor-core tiles
(:mod:`ajllm_b200.parallel.fused`); otherwise they are the collective followed/preceded by the GEMM.
The reference has no tensor parallelism; its nearest hook is the all-gather-then-GEMM in
``ajllm/training/distributed.py:76-83``.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ajllm_b200 import ops


class _GatherRows(torch.autograd.Function):
    """Forward: all-gather along dim 0. Backward: reduce-scatter (sum) along dim 0."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        size = dist.get_world_size(group)
        x = x.contiguous()
        out = torch.empty(size * x.shape[0], *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        size = dist.get_world_size(ctx.group)
        grad = grad.contiguous()
        out = torch.empty(grad.shape[0] // size, *grad.shape[1:], dtype=grad.dtype, device=grad.device)
        dist.reduce_scatter_tensor(out, grad, op=dist.ReduceOp.SUM, group=ctx.group)
        return out, None


class _ScatterRows(torch.autograd.Function):
    """Forward: reduce-scatter (sum) along dim 0. Backward: all-gather along dim 0."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        size = dist.get_world_size(group)
        x = x.contiguous()
        out = torch.empty(x.shape[0] // size, *x.shape[1:], dtype=x.dtype, device=x.device)
        dist.reduce_scatter_tensor(out, x, op=dist.ReduceOp.SUM, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        size = dist.get_world_size(ctx.group)
        grad = grad.contiguous()
        out = torch.empty(size * grad.shape[0], *grad.shape[1:], dtype=grad.dtype, device=grad.device)
        dist.all_gather_into_tensor(out, grad, group=ctx.group)
        return out, None


class TensorParallel:
    def __init__(self, group, rank: int | None = None, size: int | None = None, fused=None) -> None:
        self.group = group
        self.size = size if size is not None else (dist.get_world_size(group) if group is not None else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if group is not None else 0)
        self.fused = fused          # optional ajllm_b200.parallel.fused.FusedTensorParallel
        # one fused context per micro-batch in flight (each has its own symmetric buffers and flag words);
        # `select(i)` makes context i the one the next forward calls use (backward passes keep the one they saw)
        self.fused_contexts = [fused] if fused is not None else []

    def select(self, index: int) -> None:
        if self.fused_contexts:
            self.fused = self.fused_contexts[index % len(self.fused_contexts)]

    # ----- layout helpers
    def local_rows(self, flat: torch.Tensor) -> torch.Tensor:
        rows = flat.shape[0]
        if rows % self.size:
            raise ValueError(f"{rows} tokens cannot be split evenly over {self.size} tensor-parallel ranks")
        per = rows // self.size
        return flat[self.rank * per:(self.rank + 1) * per]

    def all_gather_cat(self, local: torch.Tensor, dim: int, differentiable: bool = False) -> torch.Tensor:
        """Concatenate every rank's ``local`` along ``dim``."""
        if self.size == 1:
            return local
        if differentiable:
            moved = local.transpose(0, dim) if dim != 0 else local
            out = _GatherRows.apply(moved.contiguous(), self.group)
            return out.transpose(0, dim) if dim != 0 else out
        pieces = [torch.empty_like(local) for _ in range(self.size)]
        dist.all_gather(pieces, local.contiguous(), group=self.group)
        return torch.cat(pieces, dim=dim)

    # ----- the two fusion points
    def gather_linear(self, x_local: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``all_gather_rows(x_local) @ weight.T`` (column-parallel)."""
        if self.fused is not None and x_local.is_cuda:
            return self.fused.gather_linear(x_local, weight)
        return ops.linear(_GatherRows.apply(x_local, self.group), weight)

    def linear_scatter(self, x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """``reduce_scatter_rows(x @ weight.T)`` (row-parallel)."""
        if self.fused is not None and x.is_cuda:
            return self.fused.linear_scatter(x, weight)
        return _ScatterRows.apply(ops.linear(x, weight), self.group)

    def swiglu_ffn(self, x_local: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
        """Sequence-parallel SwiGLU block ``reduce_scatter_rows((silu(g) * u) @ w2.T)`` with ``(g, u)`` the interleaved
        columns of ``all_gather_rows(x_local) @ w13.T``."""
        if self.fused is not None and x_local.is_cuda:
            return self.fused.swiglu_ffn(x_local, w13, w2)
        return _ScatterRows.apply(ops.swiglu_ffn(_GatherRows.apply(x_local, self.group), w13, w2), self.group)

    def all_reduce_sum_(self, tensor: torch.Tensor) -> torch.Tensor:
        if self.size > 1:
            dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=self.group)
        return tensor


def tp_optimizer_classes(tp: TensorParallel) -> list[dict]:
    """Parameter classes for :class:`ajllm_b200.training.optim.FlatAdamW` under tensor parallelism:
    sharded matrices need no gradient reduction but their norm is summed over the group; replicated
    tensors are summed over the group and counted once."""
    def sharded(name: str, p) -> bool:
        return any(name.endswith(s) for s in ("attention.qkv_proj", "attention.output_proj", "feed_forward.w13",
                                              "feed_forward.w2", "feed_forward.w1"))
    return [
        {"name": "replicated", "match": lambda n, p: not sharded(n, p), "reduce_group": tp.group, "norm_group": None},
        {"name": "tp_sharded", "match": sharded, "reduce_group": None, "norm_group": tp.group},
    ]
