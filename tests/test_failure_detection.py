"""Failure detection without faulting any device: failures are made on the host (a rank that leaves, a
corrupt file, a data source that raises) and the survivors must notice through an error, not hang."""

import datetime
import os

import pytest
import torch

from tests.conftest import free_port


def _leaver_and_survivor(rank, world, port, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=6))
    value = torch.ones(4)
    dist.all_reduce(value)                      # a healthy step first
    assert float(value[0]) == world
    if rank == 1:
        os._exit(0)                             # leaves between steps, without joining the next collective
    try:
        dist.all_reduce(torch.ones(4))
        results["survivor"] = "no error"
    except Exception as error:  # noqa: BLE001 - any error is the detection
        results["survivor"] = f"detected: {type(error).__name__}"


def test_survivor_notices_a_rank_that_left():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_leaver_and_survivor, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    assert not any(p.is_alive() for p in procs), "the survivor hung instead of failing"
    assert results.get("survivor", "").startswith("detected"), dict(results)


def test_data_source_failure_surfaces_in_the_training_loop(tmp_path):
    from ajllm_b200.training.data import BatchStager

    class Broken:
        def sample_windows(self, *args):
            raise OSError("disk went away")

    import numpy as np
    stager = BatchStager(Broken(), 2, 8, torch.device("cpu"), np.random.default_rng(0))
    with pytest.raises(OSError, match="disk went away"):
        stager.next()
    stager.close()


def test_resume_refuses_a_truncated_checkpoint(tmp_path):
    from ajllm_b200.models import build_model
    from ajllm_b200.training import FlatAdamW, load_checkpoint, save_checkpoint
    from tests.helpers import TINY_MODEL

    model = build_model(TINY_MODEL, 30)
    path = save_checkpoint(tmp_path / "latest.pt", model, FlatAdamW(model, 1e-3), 3, {})
    blob = path.read_bytes()
    path.write_bytes(blob[: len(blob) // 2])
    with pytest.raises(RuntimeError, match="unreadable"):
        load_checkpoint(path, model)
    # the atomic writer never leaves a half-written file under the final name
    assert not list(tmp_path.glob("*.tmp"))
