"""Shared pytest configuration: the ``gpu`` marker and helpers for multi-rank CPU tests."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

# the reference package as an oracle: AJLLM_REFERENCE_SRC (a directory that contains `ajllm/`), else the copy that
# the reference arm of bench.py uses; tests marked `needs_reference` are skipped when neither exists
REFERENCE_SRC = Path(os.environ.get("AJLLM_REFERENCE_SRC") or ROOT / "baseline" / "_ref")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")
    config.addinivalue_line("markers", "needs_reference: imports the reference implementation as an oracle")


def pytest_collection_modifyitems(config, items):
    import torch

    have_gpu = torch.cuda.is_available()
    have_reference = REFERENCE_SRC.is_dir()
    for item in items:
        if "gpu" in item.keywords and not have_gpu:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "needs_reference" in item.keywords and not have_reference:
            item.add_marker(pytest.mark.skip(reason="reference checkout not mounted"))


@pytest.fixture
def reference_path():
    """Puts the reference package on ``sys.path`` for the duration of a test."""
    sys.path.insert(0, str(REFERENCE_SRC))
    try:
        yield REFERENCE_SRC
    finally:
        sys.path.remove(str(REFERENCE_SRC))


def free_port() -> int:
    with socket.socket(socket.AF_INET, socket.SOCK_STREAM) as sock:
        sock.bind(("127.0.0.1", 0))
        return sock.getsockname()[1]


def run_ranks(fn, world_size: int, *args, timeout: float = 240.0):
    """Run ``fn(rank, world_size, port, *args)`` in ``world_size`` spawned CPU processes (gloo)."""
    import torch.multiprocessing as mp

    port = free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank_entry, args=(fn, rank, world_size, port, args)) for rank in range(world_size)]
    for proc in procs:
        proc.start()
    for proc in procs:
        proc.join(timeout)
    codes = []
    for proc in procs:
        if proc.is_alive():
            proc.kill()
            proc.join()
            codes.append("timeout")
        else:
            codes.append(proc.exitcode)
    assert all(code == 0 for code in codes), f"rank exit codes: {codes}"


def _rank_entry(fn, rank, world_size, port, args):
    import torch.distributed as dist

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["RANK"] = str(rank)
    os.environ["WORLD_SIZE"] = str(world_size)
    dist.init_process_group("gloo", rank=rank, world_size=world_size)
    try:
        fn(rank, world_size, *args)
    finally:
        dist.destroy_process_group()
