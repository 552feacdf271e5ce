"""Two micro-batches in flight on streams of their own (``TransformerLM.loss_interleaved``) must give the gradients
of the one-after-the-other schedule: same loss, same accumulated gradient buffer, on one GPU and, with the fused
tensor-parallel kernels and their SM budgets, on two."""

import os

import pytest
import torch

from tests.conftest import free_port

pytestmark = pytest.mark.gpu

CONFIG = {"name": "il", "context_length": 256, "d_model": 512, "num_layers": 3, "num_heads": 4, "num_kv_heads": 2,
          "d_ff": 1408, "init": {"type": "normal", "std": 0.02}}
VOCAB = 4096


def _rel(a, b):
    return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))


def _train(model, optimizer, batches, steps):
    from ajllm_b200.training import optimizer_step

    losses = []
    for step in range(steps):
        it = iter(batches[step])
        loss, norm = optimizer_step(model, optimizer, lambda: next(it), len(batches[step]), 1.0)
        losses.append(float(loss.detach()))
    torch.cuda.synchronize()
    return losses


def test_interleaved_microbatches_match_sequential_ones_on_one_gpu(monkeypatch):
    from ajllm_b200.models import build_model
    from ajllm_b200.ops import functional, native
    from ajllm_b200.training import FlatAdamW

    # reproducible kernels (no K-sliced atomic weight gradients, two-kernel attention backward): what is left to differ
    # between the two schedules is the order of a few fp32 additions
    monkeypatch.setattr(functional, "DETERMINISTIC_ATTENTION_BACKWARD", True)
    monkeypatch.setattr(functional, "DETERMINISTIC_WGRAD", True)
    device = torch.device("cuda", 0)
    gen = torch.Generator().manual_seed(3)
    steps = 3
    batches = [[torch.randint(0, VOCAB, (2, 257), generator=gen).to(device) for _ in range(4)] for _ in range(steps)]
    batches = [[(t[:, :-1], t[:, 1:]) for t in step] for step in batches]
    results = {}
    try:
        for mode in ("sequential", "interleaved"):
            torch.manual_seed(0)
            model = build_model(CONFIG, VOCAB).to(device=device, dtype=torch.bfloat16)
            model._interleave = 2 if mode == "interleaved" else 1
            optimizer = FlatAdamW(model, learning_rate=1e-4, weight_decay=0.1)
            first = _train(model, optimizer, batches[:1], 1)
            first_grad = optimizer.grad.clone()          # same weights in both modes: only the schedule differs
            losses = first + _train(model, optimizer, batches[1:], steps - 1)
            results[mode] = (losses, first_grad, optimizer.master.clone())
            assert (functional.wgrad_stream() is not None) == (mode == "interleaved")
    finally:
        functional.set_wgrad_stream(None)
    (l0, g0, w0), (l1, g1, w1) = results["sequential"], results["interleaved"]
    assert all(abs(a - b) < 2e-3 for a, b in zip(l0, l1)), (l0, l1)
    assert _rel(g1, g0) < 1e-4, _rel(g1, g0)        # a lost or doubled accumulation would show as percents
    assert _rel(w1, w0) < 2e-3, _rel(w1, w0)
    assert native.check_status() == 0


def _tp_worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from ajllm_b200.models import build_model
        from ajllm_b200.ops import functional, native
        from ajllm_b200.parallel import ParallelMesh, tp_optimizer_classes
        from ajllm_b200.parallel.contexts import make_tensor_parallel, tp_backend
        from ajllm_b200.training import FlatAdamW

        mesh = ParallelMesh(tp=world)
        gen = torch.Generator().manual_seed(3)
        steps = 3
        batches = [[torch.randint(0, VOCAB, (2, 257), generator=gen).to(device) for _ in range(4)] for _ in range(steps)]
        batches = [[(t[:, :-1], t[:, 1:]) for t in step] for step in batches]
        out = {}
        for mode, fused, interleave in (("nccl", False, 1), ("fused", True, 1), ("fused_interleaved", True, 2)):
            functional.set_wgrad_stream(None)
            tp = make_tensor_parallel(mesh.tp, device, fused=fused, interleave=interleave)
            if interleave > 1:
                for context in tp.fused_contexts:
                    context.sm_budget_mode = 48          # these tiny projections are never link-bound: force a budget
            assert tp_backend(tp) == ("fused-symmetric-memory" if fused else "nccl")
            torch.manual_seed(0)
            model = build_model(CONFIG, VOCAB, tp=tp).to(device=device, dtype=torch.bfloat16)
            assert model.interleave == interleave
            optimizer = FlatAdamW(model, learning_rate=1e-4, weight_decay=0.1, classes=tp_optimizer_classes(tp))
            losses = _train(model, optimizer, batches, steps)
            total = torch.tensor(losses, device=device)
            dist.all_reduce(total)                       # ranks hold shares of the mean loss
            out[mode] = (total.tolist(), optimizer.master.clone())
            if fused:
                assert all(context.guards_intact() for context in tp.fused_contexts)
        functional.set_wgrad_stream(None)
        report = {}
        for mode in ("fused", "fused_interleaved"):
            report[mode] = {"loss": max(abs(a - b) for a, b in zip(out[mode][0], out["nccl"][0])),
                            "weights": _rel(out[mode][1], out["nccl"][1])}
        torch.cuda.synchronize()
        results[rank] = {"report": report, "status": native.lib().ajb_check_status()}
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_interleaved_tensor_parallel_training_matches_the_nccl_path():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    results = ctx.Manager().dict()
    port = free_port()
    procs = [ctx.Process(target=_tp_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive and all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(2):
        out = results[rank]
        assert out["status"] == 0, out
        for mode, numbers in out["report"].items():
            assert numbers["loss"] < 2e-2 and numbers["weights"] < 5e-3, out       # bf16 partial sums in another order
