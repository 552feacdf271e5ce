"""Device-side timing and clock sampling.

The reference times with ``perf_counter`` after ``cuda.synchronize``
(``ajllm/workflows/benchmark_distributed.py:120-126,208-241``). Here every number comes from CUDA
events on the launching stream and, across ranks, the maximum is reported.
"""

from __future__ import annotations

import contextlib
import os
import shutil
import statistics
import subprocess
import threading
import time
from typing import Any

import torch

_QUERY = (
    "clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
    "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
    "clocks_event_reasons.sw_power_cap"
)


_NVTX = os.environ.get("AJB_NVTX", "0") == "1"


@contextlib.contextmanager
def nvtx_range(name: str):
    """Named range around a fused path (all-gather GEMM, expert dispatch, gradient reduce-scatter, ...) for a
    timeline profiler; a no-op unless ``AJB_NVTX=1`` and a GPU is present."""
    if _NVTX and torch.cuda.is_available():
        torch.cuda.nvtx.range_push(name)
        try:
            yield
        finally:
            torch.cuda.nvtx.range_pop()
    else:
        yield


class DeviceTimer:
    """Pair of CUDA events around a region; ``elapsed_ms`` synchronises on the end event."""

    def __init__(self) -> None:
        self._start = torch.cuda.Event(enable_timing=True)
        self._stop = torch.cuda.Event(enable_timing=True)

    def __enter__(self) -> "DeviceTimer":
        self._start.record()
        return self

    def __exit__(self, *exc: Any) -> None:
        self._stop.record()

    def elapsed_ms(self) -> float:
        self._stop.synchronize()
        return float(self._start.elapsed_time(self._stop))


def max_over_ranks(value: float, device: torch.device | None = None) -> float:
    """All-reduce(MAX) of a host float; identity when no process group exists."""
    import torch.distributed as dist

    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(value)
    backend = dist.get_backend()
    where = device if (device is not None and backend == "nccl") else torch.device("cpu")
    box = torch.tensor([value], dtype=torch.float64, device=where)
    dist.all_reduce(box, op=dist.ReduceOp.MAX)
    return float(box.item())


class ClockSampler:
    """Polls ``nvidia-smi`` for SM clock and throttle reasons while a timed region runs.

    Reading these values changes no GPU setting.
    """

    def __init__(self, gpu_index: int = 0, period_s: float = 0.2) -> None:
        self.gpu_index = gpu_index
        self.period_s = period_s
        self.samples: list[dict[str, Any]] = []
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def _poll_once(self) -> None:
        exe = shutil.which("nvidia-smi")
        if exe is None:
            return
        try:
            out = subprocess.run(
                [exe, f"--query-gpu={_QUERY}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index)],
                capture_output=True, text=True, timeout=5,
            ).stdout.strip()
        except (OSError, subprocess.SubprocessError):
            return
        parts = [p.strip() for p in out.split(",")]
        if len(parts) < 7:
            return
        try:
            self.samples.append({
                "sm_mhz": float(parts[0]), "sm_max_mhz": float(parts[1]), "power_w": float(parts[2]),
                "hw_slowdown": parts[3], "hw_thermal_slowdown": parts[4],
                "sw_thermal_slowdown": parts[5], "sw_power_cap": parts[6],
            })
        except ValueError:
            return

    def _loop(self) -> None:
        while not self._stop.is_set():
            self._poll_once()
            self._stop.wait(self.period_s)

    def start(self) -> "ClockSampler":
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict[str, Any]:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=10)
        return self.summary()

    def summary(self) -> dict[str, Any]:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        # "under load" = samples above half of the observed peak power
        peak = max(s["power_w"] for s in self.samples)
        loaded = [s for s in self.samples if s["power_w"] >= 0.5 * peak] or self.samples
        reasons = sorted({
            key for s in self.samples
            for key in ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
            if s[key].lower().startswith("active")
        })
        return {
            "sm_mhz": statistics.median(s["sm_mhz"] for s in loaded),
            "sm_max_mhz": max(s["sm_max_mhz"] for s in self.samples),
            "power_w_max": peak,
            "reasons": reasons,
            "samples": len(self.samples),
        }


def wall_seconds() -> float:
    return time.perf_counter()
