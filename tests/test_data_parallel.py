"""Replicated data parallelism over gloo ranks: two replicas on half batches must reproduce single-process
training on the whole batch (losses, clipped updates), with one gradient all-reduce per parameter class."""

import torch

from tests.conftest import run_ranks

CONFIG = {"name": "dp", "context_length": 16, "d_model": 32, "num_layers": 2, "num_heads": 4, "num_kv_heads": 2, "d_ff": 64,
          "tie_embeddings": True, "init": {"type": "normal", "std": 0.05}}
VOCAB = 64


def _single(tokens):
    from ajllm_b200.models import build_model
    from ajllm_b200.training.optim import FlatAdamW

    torch.manual_seed(0)
    model = build_model(CONFIG, VOCAB)
    state0 = {k: v.clone() for k, v in model.state_dict().items()}
    opt = FlatAdamW(model, 1e-2, (0.9, 0.95), 1e-8, 0.1)
    losses = []
    for batch in tokens:
        opt.zero_grad()
        loss = model.loss(batch[:, :-1], batch[:, 1:])
        loss.backward()
        opt.step(0.5)
        losses.append(float(loss.detach()))
    return state0, losses, {k: v.clone() for k, v in model.state_dict().items()}


def _rank(rank, world, state0, tokens, want_losses, want_state):
    import torch.distributed as dist

    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ParallelMesh
    from ajllm_b200.parallel.data_parallel import optimizer_classes
    from ajllm_b200.training.optim import FlatAdamW

    mesh = ParallelMesh(tp=1, fsdp=world)
    torch.manual_seed(0)
    model = build_model(CONFIG, VOCAB)
    model.load_state_dict(state0)
    model.data_parallel_share = 1.0 / world
    opt = FlatAdamW(model, 1e-2, (0.9, 0.95), 1e-8, 0.1, classes=optimizer_classes(mesh))
    for batch, want in zip(tokens, want_losses):
        per = batch.shape[0] // world
        mine = batch[rank * per:(rank + 1) * per]
        opt.zero_grad()
        loss = model.loss(mine[:, :-1], mine[:, 1:])
        loss.backward()
        opt.step(0.5)
        total = loss.detach().clone()
        dist.all_reduce(total, group=mesh.dp.group)
        assert abs(float(total) - want) < 1e-5, (float(total), want)
    for key, value in want_state.items():
        got = model.state_dict()[key]
        assert torch.allclose(got, value, atol=2e-5), (key, float((got - value).abs().max()))


def test_two_replicas_match_single_process():
    torch.manual_seed(3)
    tokens = [torch.randint(0, VOCAB, (4, 13)) for _ in range(2)]
    state0, losses, state1 = _single(tokens)
    run_ranks(_rank, 2, state0, tokens, losses, state1)
