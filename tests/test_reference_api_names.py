"""The reference's public names resolve to this package's implementations."""

import torch

from tests.conftest import run_ranks


def test_device_and_seed_helpers_keep_the_reference_names():
    from ajllm_b200 import utils

    assert utils.resolve_device("cpu") == torch.device("cpu")
    assert utils.resolve_device is utils.pick_device and utils.seed_everything is utils.seed_all
    utils.seed_everything(7)
    first = torch.rand(3)
    utils.seed_everything(7)
    assert torch.equal(first, torch.rand(3))
    assert utils.explain_device_selection("cpu", torch.device("cpu")) is None


def test_console_scripts_include_the_reference_name():
    import tomllib
    from pathlib import Path

    scripts = tomllib.loads((Path(__file__).resolve().parent.parent / "pyproject.toml").read_text())["project"]["scripts"]
    assert scripts["ajllm"] == scripts["ajllm-b200"] == "ajllm_b200.cli:main"


def _sharded_by_reference_name(rank, world):
    from ajllm_b200.models import build_model
    from ajllm_b200.training.distributed import FullyShardedDataParallel
    from tests.helpers import TINY_MODEL

    torch.manual_seed(0)
    plain = build_model(TINY_MODEL, 40)
    want = {k: v.clone() for k, v in plain.state_dict().items()}
    model = FullyShardedDataParallel(plain, compute_dtype=None, activation_checkpointing=True, learning_rate=1e-2)
    full = model.gather_full_params()
    assert list(full) == list(want) and all(torch.equal(full[k], want[k]) for k in want)
    tokens = torch.randint(0, 40, (2, 17), generator=torch.Generator().manual_seed(rank))
    model.optimizer.zero_grad()
    loss = model.loss(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    model.finish_gradient_synchronization()
    model.optimizer.step(1.0)
    after = model.gather_full_params()
    assert any(not torch.equal(after[k], want[k]) for k in want)


def test_fully_sharded_data_parallel_adapter_trains_over_two_ranks():
    run_ranks(_sharded_by_reference_name, 2)
