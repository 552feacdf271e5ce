"""Process mesh over ``torch.distributed``: tensor, expert, fully-sharded-data and pipeline axes.

The reference only ever uses the default world group (``ajllm/workflows/lm_train.py:95-103``). Here
ranks are laid out ``rank = (pp_index * fsdp + dp_index) * tp + tp_index`` so that the
tensor-parallel peers (the chattiest axis) are adjacent GPUs; expert-parallel groups are runs of
``ep`` consecutive data-parallel ranks. Backend: ``nccl`` on CUDA, ``gloo`` on CPU.
"""

from __future__ import annotations

import datetime
import os
from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist


def init_distributed(device_type: str = "auto", timeout_s: float | None = None) -> tuple[int, int, torch.device]:
    """Join the env:// rendezvous when launched by torchrun; returns ``(rank, world, device)``. The process-group
    timeout is ``timeout_s``, else ``AJB_DIST_TIMEOUT_S``, else 30 minutes."""
    if timeout_s is None:
        timeout_s = float(os.environ.get("AJB_DIST_TIMEOUT_S", "1800"))
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    use_cuda = torch.cuda.is_available() if device_type == "auto" else device_type == "cuda"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kwargs: dict[str, Any] = {"timeout": datetime.timedelta(seconds=timeout_s)}
        if use_cuda:
            kwargs["device_id"] = device
        dist.init_process_group("nccl" if use_cuda else "gloo", rank=rank, world_size=world, **kwargs)
    return rank, world, device


@dataclass
class AxisGroup:
    """One rank's view of a mesh axis."""

    group: Any
    rank: int
    size: int
    ranks: list[int] = field(default_factory=list)


class ParallelMesh:
    def __init__(self, tp: int = 1, fsdp: int | None = None, ep: int = 1, pp: int = 1) -> None:
        self.world = dist.get_world_size() if dist.is_initialized() else 1
        self.rank = dist.get_rank() if dist.is_initialized() else 0
        fsdp = fsdp if fsdp is not None else max(1, self.world // (tp * pp))
        if tp * fsdp * pp != self.world:
            raise ValueError(f"mesh tp={tp} x fsdp={fsdp} x pp={pp} does not cover {self.world} ranks")
        if fsdp % ep:
            raise ValueError("ep must divide fsdp")
        self.tp_size, self.dp_size, self.ep_size, self.pp_size = tp, fsdp, ep, pp
        self.tp_index = self.rank % tp
        self.dp_index = (self.rank // tp) % fsdp
        self.pp_index = self.rank // (tp * fsdp)
        self.tp = self._axis([[(p * fsdp + d) * tp + t for t in range(tp)] for p in range(pp) for d in range(fsdp)])
        self.dp = self._axis([[(p * fsdp + d) * tp + t for d in range(fsdp)] for p in range(pp) for t in range(tp)])
        self.pp = self._axis([[(p * fsdp + d) * tp + t for p in range(pp)] for d in range(fsdp) for t in range(tp)])
        self.ep = self._axis([[(p * fsdp + d0 + e) * tp + t for e in range(ep)]
                              for p in range(pp) for t in range(tp) for d0 in range(0, fsdp, ep)])
        # replicas of an expert shard: same position inside the EP group, different EP groups
        self.ep_replica = self._axis([[(p * fsdp + d0 + e) * tp + t for d0 in range(0, fsdp, ep)]
                                      for p in range(pp) for t in range(tp) for e in range(ep)])

    def _axis(self, groups: list[list[int]]) -> AxisGroup:
        mine = None
        for ranks in groups:
            handle = None
            if self.world > 1 and len(ranks) > 1:
                handle = dist.new_group(ranks)      # every rank must create every group
            if self.rank in ranks:
                mine = AxisGroup(handle, ranks.index(self.rank), len(ranks), ranks)
        assert mine is not None
        return mine
