"""The reference's entry point for sharded training, under its own name and signature.

``ajllm/training/distributed.py:164-379`` exposes ``FullyShardedDataParallel(module, compute_dtype,
activation_checkpointing)`` with ``finish_gradient_synchronization()`` and ``gather_full_params()``.
Code written against that surface runs on :class:`ajllm_b200.parallel.fsdp.ShardedDataParallel`
through this adapter: the world group is the shard group, ``compute_dtype`` casts the wrapped module
once (master weights and optimizer state stay fp32 inside the wrapper), and activation checkpointing
is per transformer block. Differences that a caller can see: the wrapper owns its optimizer
(``.optimizer``, AdamW over the shards), ``loss(inputs, targets)`` runs forward and backward unit by
unit (``forward`` alone returns logits for evaluation), and gradients of every parameter are already
reduced when ``loss(...).backward()`` returns, so ``finish_gradient_synchronization`` has nothing left
to do.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

from ajllm_b200.parallel.fsdp import ShardedDataParallel


class FullyShardedDataParallel(ShardedDataParallel):
    def __init__(self, module: torch.nn.Module, compute_dtype: torch.dtype | None = None,
                 activation_checkpointing: bool = True, **optimizer_options) -> None:
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("FullyShardedDataParallel needs an initialised torch.distributed process group")
        if compute_dtype is not None:
            if compute_dtype == torch.float16:
                compute_dtype = torch.bfloat16      # same fp32 master weights, wider exponent, no loss scaling
            module = module.to(dtype=compute_dtype)
        super().__init__(module, dist.group.WORLD, checkpoint_layers=activation_checkpointing, **optimizer_options)
        self.compute_dtype = compute_dtype
        self.activation_checkpointing = activation_checkpointing

    def finish_gradient_synchronization(self) -> None:
        """Kept for callers of the reference API: every gradient (sharded matrices through the reduce-scatter of
        their unit, norm gains with them) is complete when the backward pass of ``loss`` returns."""

    def gather_full_params(self) -> dict[str, torch.Tensor]:
        """Un-sharded fp32 parameters under the model's checkpoint key names (a collective: every rank calls it)."""
        return self.export_named(self.master, self.local_master)
