"""Tensor parallelism over gloo ranks: a 2-rank model must reproduce the single-process model."""

import torch

from tests.conftest import run_ranks

CONFIG = {"name": "cfg1", "context_length": 128, "d_model": 256, "num_layers": 4, "num_heads": 8, "num_kv_heads": 4,
          "d_ff": 688, "tie_embeddings": True, "position_encoding": {"type": "rope", "theta": 10000},
          "init": {"type": "normal", "std": 0.02}}
VOCAB = 8192


def _single_process_step():
    from ajllm_b200.models import build_model
    from ajllm_b200.training.optim import FlatAdamW

    torch.manual_seed(0)
    model = build_model(CONFIG, VOCAB)
    state0 = {k: v.clone() for k, v in model.state_dict().items()}
    gen = torch.Generator().manual_seed(1)
    tokens = torch.randint(0, VOCAB, (4, 129), generator=gen)
    opt = FlatAdamW(model, learning_rate=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    opt.zero_grad()
    loss = model.loss(tokens[:, :-1], tokens[:, 1:])
    loss.backward()
    norm = opt.step(1.0)
    return state0, tokens, float(loss), float(norm), {k: v.clone() for k, v in model.state_dict().items()}


def _tp_rank(rank, world, state0, tokens, want_loss, want_norm, want_state):
    import torch.distributed as dist

    from ajllm_b200.models import build_model
    from ajllm_b200.parallel import ParallelMesh, TensorParallel, tp_optimizer_classes
    from ajllm_b200.training.optim import FlatAdamW

    mesh = ParallelMesh(tp=world)
    tp = TensorParallel(mesh.tp.group, mesh.tp.rank, mesh.tp.size)
    torch.manual_seed(0)
    model = build_model(CONFIG, VOCAB, tp=tp)
    model.load_state_dict(state0)
    opt = FlatAdamW(model, learning_rate=3e-4, betas=(0.9, 0.95), weight_decay=0.1, classes=tp_optimizer_classes(tp))
    opt.zero_grad()
    share = model.loss(tokens[:, :-1], tokens[:, 1:])
    share.backward()
    norm = opt.step(1.0)
    total = share.detach().clone()
    dist.all_reduce(total)
    assert abs(float(total) - want_loss) < 1e-4, (float(total), want_loss)
    assert abs(float(norm) - want_norm) < 1e-4 * max(1.0, want_norm), (float(norm), want_norm)
    got = model.state_dict()
    for key, value in want_state.items():
        assert torch.allclose(got[key], value, atol=2e-5, rtol=1e-4), key
    # logits path gathers all tokens on every rank
    logits = model(tokens[:, :-1])
    assert logits.shape == (4, 128, VOCAB)


def test_two_rank_tensor_parallel_matches_single_process():
    state0, tokens, loss, norm, state1 = _single_process_step()
    run_ranks(_tp_rank, 2, state0, tokens, loss, norm, state1)
