"""Context parallelism over gloo ranks: two ranks holding half of every sequence (heads traded by all-to-all inside
attention) must reproduce single-process training on whole sequences: loss, logits, updated weights."""

import pytest
import torch

from tests.conftest import run_ranks

CONFIG = {"name": "cp", "context_length": 16, "d_model": 32, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2, "d_ff": 64,
          "init": {"type": "normal", "std": 0.05}}
LEARNED = {**CONFIG, "position_encoding": {"type": "learned"}, "num_kv_heads": 4}
VOCAB = 64


def _single(config, tokens):
    from ajllm_b200.models import build_model
    from ajllm_b200.training.optim import FlatAdamW

    torch.manual_seed(0)
    model = build_model(config, VOCAB)
    state0 = {k: v.clone() for k, v in model.state_dict().items()}
    with torch.no_grad():
        logits = model(tokens[0][:, :-1]).clone()
    opt = FlatAdamW(model, 1e-2, (0.9, 0.95), 1e-8, 0.1)
    losses = []
    for batch in tokens:
        opt.zero_grad()
        loss = model.loss(batch[:, :-1], batch[:, 1:])
        loss.backward()
        opt.step(0.5)
        losses.append(float(loss.detach()))
    return state0, logits, losses, {k: v.clone() for k, v in model.state_dict().items()}


def _rank(rank, world, config, state0, tokens, want_logits, want_losses, want_state):
    import torch.distributed as dist

    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ContextParallel, ParallelMesh
    from ajllm_b200.parallel.data_parallel import optimizer_classes
    from ajllm_b200.training.optim import FlatAdamW

    mesh = ParallelMesh(tp=world, fsdp=1)           # the context-parallel group takes the innermost axis
    cp = ContextParallel(mesh.tp.group, mesh.tp.rank, mesh.tp.size)
    torch.manual_seed(0)
    model = build_model(config, VOCAB, cp=cp)
    model.load_state_dict(state0)
    with torch.no_grad():
        logits = model(tokens[0][:, :-1])
    assert torch.allclose(logits, want_logits, atol=2e-5), float((logits - want_logits).abs().max())
    opt = FlatAdamW(model, 1e-2, (0.9, 0.95), 1e-8, 0.1, classes=optimizer_classes(mesh, None, cp))
    for batch, want in zip(tokens, want_losses):
        opt.zero_grad()
        loss = model.loss(batch[:, :-1], batch[:, 1:])       # every rank gets whole sequences and keeps its slice
        loss.backward()
        opt.step(0.5)
        total = loss.detach().clone()
        dist.all_reduce(total, group=cp.group)
        assert abs(float(total) - want) < 1e-5, (float(total), want)
    for key, value in want_state.items():
        got = model.state_dict()[key]
        assert torch.allclose(got, value, atol=1e-4), (key, float((got - value).abs().max()))


@pytest.mark.parametrize("config", [CONFIG, LEARNED])
def test_two_context_parallel_ranks_match_single_process(config):
    torch.manual_seed(3)
    tokens = [torch.randint(0, VOCAB, (3, 17)) for _ in range(2)]
    state0, logits, losses, state1 = _single(config, tokens)
    run_ranks(_rank, 2, config, state0, tokens, logits, losses, state1)


def test_parallel_config_accepts_cp_with_data_parallelism_only():
    from ajllm_b200.config import ConfigError, check_parallel

    assert check_parallel({"cp": 2}, 4) == {"tp": 1, "ep": 1, "fsdp": 2, "pp": 1, "cp": 2}
    with pytest.raises(ConfigError):
        check_parallel({"cp": 2, "tp": 2}, 4)
