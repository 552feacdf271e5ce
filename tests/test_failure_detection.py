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


def _tiny_trainer(tmp_path, validation: bool = False, device=None, model=None, optimizer=None, **kwargs):
    from ajllm_b200.models import build_model
    from ajllm_b200.training.data import SyntheticTokens
    from ajllm_b200.training.trainer import Trainer
    from tests.helpers import TINY_MODEL

    model = model if model is not None else build_model(TINY_MODEL, 30)
    config = {"training": {"batch_size": 2, "max_steps": 2}, "optimizer": {"max_lr": 1e-3},
              "logging": {"log_interval": 1, "eval_interval": 0, "eval_batches": 1, "checkpoint_interval": 1}}
    data = SyntheticTokens(30, length=4096, seed=1)
    return Trainer(model, data, data if validation else None, tmp_path, config, device or torch.device("cpu"), 0,
                   optimizer=optimizer, **kwargs)


def test_a_kernel_timeout_stops_training_before_any_checkpoint_is_written(tmp_path, monkeypatch):
    from ajllm_b200.ops import native
    from ajllm_b200.training.trainer import Trainer

    trainer = _tiny_trainer(tmp_path)

    def timed_out(self):
        raise native.PeerTimeout(0x1e0a)
    monkeypatch.setattr(Trainer, "_check_kernels", timed_out)
    with pytest.raises(native.PeerTimeout):
        trainer.train({})
    assert not list((tmp_path / "checkpoints").glob("*.pt"))


def test_the_status_words_are_read_on_a_cuda_device(monkeypatch):
    from ajllm_b200.ops import native
    from ajllm_b200.training.trainer import Trainer

    calls = []
    monkeypatch.setattr(native, "check_status", lambda: calls.append(1))
    trainer = object.__new__(Trainer)
    trainer.device = torch.device("cpu")
    trainer._check_kernels()
    assert not calls
    trainer.device = torch.device("cuda", 0)
    trainer._check_kernels()
    assert calls == [1]


def _fsdp_without_validation(rank, world, directory):
    from pathlib import Path

    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ParallelMesh
    from ajllm_b200.parallel.fsdp import ShardedDataParallel
    from tests.helpers import TINY_MODEL

    mesh = ParallelMesh(tp=1, fsdp=world)
    torch.manual_seed(0)
    model = ShardedDataParallel(build_model(TINY_MODEL, 30), mesh.dp.group, learning_rate=1e-3)
    trainer = _tiny_trainer(Path(directory), model=model, optimizer=model.optimizer, data_rank=rank, data_world=world,
                            loss_reduce_group=mesh.dp.group)
    summary = trainer.train({})
    assert summary["status"] == "completed"
    if rank == 0:
        names = {p.name for p in (Path(directory) / "checkpoints").iterdir()}
        assert {"final.pt", "latest.pt", "best.pt"} <= names, names


def test_sharded_training_without_a_validation_split_finishes_and_writes_best(tmp_path):
    from tests.conftest import run_ranks

    run_ranks(_fsdp_without_validation, 2, str(tmp_path), timeout=120.0)
