"""Builds the tensor- and expert-parallel contexts that models are constructed with.

One place decides whether a projection and its collective run as one kernel over symmetric NVLink
memory (:mod:`ajllm_b200.parallel.fused`, :mod:`ajllm_b200.parallel.moe_exchange`) or as the NCCL
collective next to the GEMM, so the training workflow, the generation workflow and the benchmarks
cannot drift apart. On CUDA the fused kernels are the default; ``fused=False`` (the
``acceleration.fused: false`` config key) or ``AJB_FUSED_TP=0`` / ``AJB_FUSED_EP=0`` select the NCCL
composition, which is also what CPU (gloo) ranks always use. The reference has neither form of
parallelism; its nearest hook is the gather-then-GEMM of ``ajllm/training/distributed.py:76-83``.
"""

from __future__ import annotations

import os

import torch

from ajllm_b200.parallel.mesh import AxisGroup
from ajllm_b200.parallel.tensor_parallel import TensorParallel


def _wants_fused(fused: bool | None, device: torch.device, size: int, switch: str) -> bool:
    if device.type != "cuda" or not 2 <= size <= 8:
        return False
    if os.environ.get(switch, "1") == "0":
        return False
    return True if fused is None else bool(fused)


def interleaved_microbatches(tp_size: int, device: torch.device) -> int:
    """How many micro-batches a tensor-parallel training step keeps in flight on streams of their own
    (``AJB_TP_INTERLEAVE=2`` switches it on). Off by default: measured on two and four GPUs the two streams run in
    step with each other (both in a link-bound projection, then both in attention), so the step time did not change
    (within 1 %), and an unchanged time does not pay for the second set of symmetric buffers."""
    if device.type != "cuda":
        return 1
    forced = os.environ.get("AJB_TP_INTERLEAVE")
    if forced is not None:
        return max(1, int(forced))
    return 1


def make_tensor_parallel(axis: AxisGroup, device: torch.device, fused: bool | None = None,
                         interleave: int | None = None) -> TensorParallel | None:
    """Context for ``axis`` (``None`` when the axis has one rank). A failure to set up the symmetric buffers
    raises: a GPU run does not silently fall back to the slower composition. ``interleave`` (default: by group size)
    creates that many fused contexts so that micro-batches on different streams never share buffers or flags."""
    if axis.size <= 1:
        return None
    if not _wants_fused(fused, device, axis.size, "AJB_FUSED_TP"):
        return TensorParallel(axis.group, axis.rank, axis.size)
    from ajllm_b200.parallel.fused import FusedTensorParallel
    count = interleave if interleave is not None else interleaved_microbatches(axis.size, device)
    contexts = [FusedTensorParallel(axis.group, device) for _ in range(max(1, count))]
    if len(contexts) > 1:
        # two fused kernels (one per micro-batch stream) must be resident together on every rank, whatever order the
        # hardware picks them in: each gets at most half of the device
        for context in contexts:
            context.sm_cap = context._sms // 2 // 2 * 2 - 2
    tp = TensorParallel(axis.group, axis.rank, axis.size, fused=contexts[0])
    tp.fused_contexts = contexts
    tp.interleave = len(contexts)
    # weight-gradient GEMMs leave the critical path: they run beside the link-bound fused projections
    from ajllm_b200.ops import functional
    if functional.wgrad_stream() is None and os.environ.get("AJB_WGRAD_STREAM", "1") != "0":
        functional.set_wgrad_stream(torch.cuda.Stream(device=device))
    return tp


def make_expert_parallel(axis: AxisGroup, device: torch.device, fused: bool | None = None) -> TensorParallel | None:
    """Expert-parallel context; with ``fused`` the dispatch / combine exchanges are one-kernel peer-memory transfers."""
    if axis.size <= 1:
        return None
    ep = TensorParallel(axis.group, axis.rank, axis.size)
    if _wants_fused(fused, device, axis.size, "AJB_FUSED_EP"):
        from ajllm_b200.parallel.moe_exchange import FusedExpertExchange
        ep.exchange = FusedExpertExchange(axis.group, device)
    return ep


def tp_backend(tp: TensorParallel | None) -> str:
    if tp is None or tp.size <= 1:
        return "none"
    return "fused-symmetric-memory" if tp.fused is not None else "nccl"


def expert_exchange_backend(ep: TensorParallel | None) -> str:
    if ep is None or ep.size <= 1:
        return "none"
    return "fused-symmetric-memory" if getattr(ep, "exchange", None) is not None else "nccl-all-to-all"
