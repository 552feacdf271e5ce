"""Device selection (reference: ``ajllm/utils/device.py:8-25``).

``auto`` resolves to CUDA when a GPU is visible and to the CPU otherwise. The CPU path runs the
plain PyTorch oracle math of every op; the CUDA path runs the sm_100a kernels.
"""

from __future__ import annotations

import torch


def pick_device(requested: str = "auto") -> torch.device:
    if requested and requested != "auto":
        return torch.device(requested)
    if torch.cuda.is_available():
        return torch.device("cuda", torch.cuda.current_device())
    mps = getattr(torch.backends, "mps", None)
    if mps is not None and mps.is_available():
        return torch.device("mps")
    return torch.device("cpu")


def describe_device_choice(requested: str, chosen: torch.device) -> str | None:
    """One sentence on why ``auto`` ended on the CPU, or ``None`` when there is nothing to say."""
    if requested != "auto" or chosen.type != "cpu":
        return None
    if torch.version.cuda is None:
        return "no CUDA: this PyTorch build was compiled without CUDA support"
    return "no CUDA: PyTorch has CUDA support but no GPU is visible to this process"
