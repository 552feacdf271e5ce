"""Token datasets and batch staging.

``TokenDataset`` keeps the reference's contract (``ajllm/training/data.py:11-38``): a native-endian
``uint32`` file is memory-mapped and ``batch()`` draws ``batch_size`` random windows of
``context_length + 1`` tokens, returning int64 ``(inputs, targets)`` on the device. ``BatchStager``
adds what the reference lacks: windows are gathered into pinned host memory by a worker thread and
copied to the GPU on a side stream, so the host gather and the H2D copy of step ``i+1`` overlap the
compute of step ``i``.
"""

from __future__ import annotations

import queue
import threading
from pathlib import Path

import numpy as np
import torch


class TokenDataset:
    def __init__(self, path: str | Path) -> None:
        self.path = Path(path)
        if self.path.stat().st_size % 4 != 0:
            raise ValueError(f"Token file size is not divisible by four bytes: {self.path}")
        self.tokens = np.memmap(self.path, dtype=np.uint32, mode="r")

    def __len__(self) -> int:
        return int(self.tokens.shape[0])

    def sample_windows(self, batch_size: int, context_length: int, generator: np.random.Generator) -> np.ndarray:
        """``[batch_size, context_length + 1]`` int64 windows at uniformly random offsets."""
        last_start = len(self) - context_length - 1
        if last_start < 0:
            raise ValueError(f"Dataset {self.path} has {len(self)} tokens, fewer than context_length + 1")
        starts = generator.integers(0, last_start + 1, size=batch_size)
        offsets = starts[:, None] + np.arange(context_length + 1)[None, :]
        return self.tokens[offsets].astype(np.int64)

    def batch(self, batch_size: int, context_length: int, device: torch.device,
              generator: np.random.Generator) -> tuple[torch.Tensor, torch.Tensor]:
        windows = torch.from_numpy(self.sample_windows(batch_size, context_length, generator))
        inputs, targets = windows[:, :-1].contiguous(), windows[:, 1:].contiguous()
        return inputs.to(device), targets.to(device)


class SyntheticTokens:
    """Uniform-random token ids with the ``TokenDataset`` interface (benchmarks, smoke runs)."""

    def __init__(self, vocab_size: int, length: int = 1 << 24, seed: int = 0) -> None:
        self.vocab_size = vocab_size
        self._length = length
        self.tokens = np.random.default_rng(seed).integers(0, vocab_size, size=length, dtype=np.uint32)

    def __len__(self) -> int:
        return self._length

    sample_windows = TokenDataset.sample_windows
    batch = TokenDataset.batch
    path = Path("<synthetic>")


class BatchStager:
    """Double-buffered ``(inputs, targets)`` producer over pinned memory and a copy stream."""

    def __init__(self, dataset, batch_size: int, context_length: int, device: torch.device,
                 generator: np.random.Generator, depth: int = 2) -> None:
        self.dataset, self.batch_size, self.context_length = dataset, batch_size, context_length
        self.device, self.generator = device, generator
        self.cuda = device.type == "cuda"
        self.h2d_bytes_per_batch = 2 * batch_size * context_length * 8
        self._queue: queue.Queue = queue.Queue(maxsize=depth)
        self._halt = threading.Event()
        self._copy_stream = torch.cuda.Stream(device=device) if self.cuda else None
        self._thread = threading.Thread(target=self._produce, daemon=True)
        self._thread.start()

    def _produce(self) -> None:
        try:
            while not self._halt.is_set():
                windows = torch.from_numpy(self.dataset.sample_windows(self.batch_size, self.context_length,
                                                                       self.generator))
                inputs, targets = windows[:, :-1].contiguous(), windows[:, 1:].contiguous()
                if self.cuda:
                    inputs, targets = inputs.pin_memory(), targets.pin_memory()
                while not self._halt.is_set():
                    try:
                        self._queue.put((inputs, targets), timeout=0.1)
                        break
                    except queue.Full:
                        continue
        except Exception as error:  # surfaced to the consumer
            self._queue.put(error)

    def next(self) -> tuple[torch.Tensor, torch.Tensor]:
        item = self._queue.get()
        if isinstance(item, Exception):
            raise item
        inputs, targets = item
        if not self.cuda:
            return inputs, targets
        with torch.cuda.stream(self._copy_stream):
            dev_inputs = inputs.to(self.device, non_blocking=True)
            dev_targets = targets.to(self.device, non_blocking=True)
        torch.cuda.current_stream().wait_stream(self._copy_stream)
        dev_inputs.record_stream(torch.cuda.current_stream())
        dev_targets.record_stream(torch.cuda.current_stream())
        return dev_inputs, dev_targets

    def close(self) -> None:
        self._halt.set()
        try:
            while True:
                self._queue.get_nowait()
        except queue.Empty:
            pass
        self._thread.join(timeout=5)
