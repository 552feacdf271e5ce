"""Pipeline parallelism over gloo ranks (1F1B, 2 and 3 stages) must reproduce single-process training:
losses, clipped updates and the gathered whole-model state."""

import pytest
import torch

from tests.conftest import run_ranks

CONFIG = {"name": "p", "context_length": 16, "d_model": 32, "num_layers": 4, "num_heads": 4, "num_kv_heads": 2, "d_ff": 64,
          "tie_embeddings": False, "init": {"type": "normal", "std": 0.05}}
VOCAB = 64


def _single(tokens, steps):
    from ajllm_b200.models import build_model
    from ajllm_b200.training.optim import FlatAdamW

    torch.manual_seed(0)
    model = build_model(CONFIG, VOCAB)
    state0 = {k: v.clone() for k, v in model.state_dict().items()}
    opt = FlatAdamW(model, 1e-2, (0.9, 0.95), 1e-8, 0.1)
    losses = []
    for step in range(steps):
        opt.zero_grad()
        loss = model.loss(tokens[step][:, :-1], tokens[step][:, 1:])
        loss.backward()
        opt.step(0.5)
        losses.append(float(loss))
    return state0, losses, {k: v.clone() for k, v in model.state_dict().items()}


def _rank(rank, world, state0, tokens, want_losses, want_state, microbatches):
    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ParallelMesh, PipelineParallel, pp_optimizer_classes
    from ajllm_b200.training.optim import FlatAdamW

    mesh = ParallelMesh(tp=1, fsdp=1, pp=world)
    torch.manual_seed(0)
    model = build_model(CONFIG, VOCAB)
    model.load_state_dict(state0)
    pipe = PipelineParallel(model, mesh.pp.group, microbatches)
    opt = FlatAdamW(pipe.module, 1e-2, (0.9, 0.95), 1e-8, 0.1, classes=pp_optimizer_classes(mesh.pp.group))
    for step, want in enumerate(want_losses):
        opt.zero_grad()
        loss = pipe.loss(tokens[step][:, :-1], tokens[step][:, 1:])
        loss.backward()                      # a no-op: the schedule has already back-propagated
        opt.step(0.5)
        assert abs(float(loss) - want) < 1e-5, (step, float(loss), want)
    merged = pipe.state_dict_global()
    assert set(merged) == set(want_state)
    for key, value in want_state.items():
        assert torch.allclose(merged[key], value, atol=2e-5), (key, float((merged[key] - value).abs().max()))
    with torch.no_grad():
        again = pipe.loss(tokens[0][:, :-1], tokens[0][:, 1:])
    assert torch.isfinite(again)


@pytest.mark.parametrize("world,microbatches", [(2, 4), (3, 2), (2, 1)])
def test_pipeline_training_matches_single_process(world, microbatches):
    torch.manual_seed(1)
    steps = 2
    tokens = [torch.randint(0, VOCAB, (4, 13)) for _ in range(steps)]
    state0, losses, state1 = _single(tokens, steps)
    run_ranks(_rank, world, state0, tokens, losses, state1, microbatches)


def _resume_rank(rank, world, state0, tokens, want_state):
    """Two steps, a checkpoint of whole-model weights and optimizer state in between, into fresh objects."""
    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ParallelMesh, PipelineOptimizer, PipelineParallel

    mesh = ParallelMesh(tp=1, fsdp=1, pp=world)

    def fresh(weights):
        torch.manual_seed(0)
        model = build_model(CONFIG, VOCAB)
        pipe = PipelineParallel(model, mesh.pp.group, 2)
        pipe.load_state_dict(weights)
        return pipe, PipelineOptimizer(pipe, learning_rate=1e-2, betas=(0.9, 0.95), epsilon=1e-8, weight_decay=0.1)

    pipe, opt = fresh(state0)
    opt.zero_grad()
    pipe.loss(tokens[0][:, :-1], tokens[0][:, 1:])
    opt.step(0.5)
    saved_model, saved_opt = pipe.state_dict(), opt.state_dict()
    assert list(saved_opt["param_names"]) == list(saved_model.keys())        # single-process layout
    pipe2, opt2 = fresh(saved_model)
    opt2.load_state_dict(saved_opt)
    assert opt2.step_count == 1
    opt2.zero_grad()
    pipe2.loss(tokens[1][:, :-1], tokens[1][:, 1:])
    opt2.step(0.5)
    merged = pipe2.state_dict()
    for key, value in want_state.items():
        assert torch.allclose(merged[key], value, atol=2e-5), (key, float((merged[key] - value).abs().max()))


def test_pipeline_checkpoint_round_trip_matches_uninterrupted_training():
    torch.manual_seed(1)
    tokens = [torch.randint(0, VOCAB, (4, 13)) for _ in range(2)]
    state0, _, state1 = _single(tokens, 2)
    run_ranks(_resume_rank, 2, state0, tokens, state1)
