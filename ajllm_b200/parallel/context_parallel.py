"""Context parallelism for long sequences (DeepSpeed-Ulysses style): every rank of the group holds the same
parameters and a contiguous ``T / cp`` slice of every sequence; inside attention an all-to-all trades the sequence
split for a head split (each rank then sees whole sequences for ``heads / cp`` heads, so the unmodified causal flash
kernel and its RoPE positions apply), and a second all-to-all trades back before the output projection. Norms,
projections, the feed-forward block and the loss run on the local tokens only. Parameter gradients are summed over
the group like those of data-parallel replicas.

The reference has no long-context mechanism beyond its single-GPU flash kernel
(``ajllm/modeling/flash_attention.py``); this is the extension the parallel layer offers for sequences whose
activations do not fit one GPU. The exchanges are NCCL (gloo on CPUs) ``all_to_all_single`` calls.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ajllm_b200.parallel.tensor_parallel import TensorParallel


class _AllToAll(torch.autograd.Function):
    """``out[s] = x_of_rank_s[my_rank]`` over dim 0 (equal splits); its own transpose, hence its own backward."""

    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        x = x.contiguous()
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x, group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous()
        out = torch.empty_like(grad)
        dist.all_to_all_single(out, grad, group=ctx.group)
        return out, None


class ContextParallel(TensorParallel):
    """Group helper (``rank``, ``size``, gathers) plus the two attention exchanges."""

    def local_sequence(self, x: torch.Tensor, dim: int = 1) -> torch.Tensor:
        """This rank's contiguous slice of the sequence dimension."""
        length = x.shape[dim]
        if length % self.size:
            raise ValueError(f"sequence length {length} cannot be split over {self.size} context-parallel ranks")
        per = length // self.size
        return x.narrow(dim, self.rank * per, per)

    def check_heads(self, num_heads: int, num_kv_heads: int) -> None:
        if num_heads % self.size or num_kv_heads % self.size:
            raise ValueError("the context-parallel size must divide both head counts")

    def to_heads(self, qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int) -> torch.Tensor:
        """Packed ``[B, T / cp, (Hq + 2 Hkv) * hd]`` of all heads -> ``[B, T, (Hq + 2 Hkv) / cp * hd]`` of this
        rank's heads (packed q | k | v again), whole sequences."""
        B, Tl, _ = qkv.shape
        cp = self.size
        nq, nk = num_heads * head_dim, num_kv_heads * head_dim
        q = qkv[..., :nq].reshape(B, Tl, cp, nq // cp)
        k = qkv[..., nq:nq + nk].reshape(B, Tl, cp, nk // cp)
        v = qkv[..., nq + nk:].reshape(B, Tl, cp, nk // cp)
        send = torch.cat((q, k, v), dim=-1).permute(2, 0, 1, 3)            # [cp (destination), B, Tl, Wl]
        recv = _AllToAll.apply(send, self.group)                           # [cp (source = sequence chunk), B, Tl, Wl]
        return recv.permute(1, 0, 2, 3).reshape(B, cp * Tl, -1)

    def to_sequence(self, attended: torch.Tensor, num_heads: int, head_dim: int) -> torch.Tensor:
        """``[B, T, Hq / cp * hd]`` of this rank's heads -> ``[B, T / cp, Hq * hd]`` of all heads, local tokens."""
        B, T, width = attended.shape
        cp = self.size
        Tl = T // cp
        send = attended.reshape(B, cp, Tl, width).permute(1, 0, 2, 3)      # [cp (destination chunk), B, Tl, Hl * hd]
        recv = _AllToAll.apply(send, self.group)                           # [cp (source = head chunk), B, Tl, Hl * hd]
        return recv.permute(1, 2, 0, 3).reshape(B, Tl, cp * width)
