"""Pipeline parallelism on 2 GPUs (NCCL point-to-point): two 1F1B steps must track the same model trained on
one GPU. Ranks are child processes, one per GPU."""

import os

import pytest
import torch

from tests.conftest import free_port

pytestmark = pytest.mark.gpu

MODEL = {"name": "p", "context_length": 256, "d_model": 256, "num_layers": 4, "num_heads": 2, "num_kv_heads": 1, "d_ff": 512,
         "tie_embeddings": False, "init": {"type": "normal", "std": 0.05}}
VOCAB = 512


def _worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from ajllm_b200.models import build_model
        from ajllm_b200.ops import native
        from ajllm_b200.parallel import ParallelMesh, PipelineParallel, pp_optimizer_classes
        from ajllm_b200.training.optim import FlatAdamW

        def batches(step):
            gen = torch.Generator().manual_seed(500 + step)
            return torch.randint(0, VOCAB, (8, 129), generator=gen).to(device)

        # one-GPU run of the same model (every rank computes it: same seed, same data)
        torch.manual_seed(0)
        with torch.device(device):
            whole = build_model(MODEL, VOCAB).to(dtype=torch.bfloat16)
        state0 = {k: v.clone() for k, v in whole.state_dict().items()}
        opt = FlatAdamW(whole, 1e-3, (0.9, 0.95), 1e-8, 0.0)
        want = []
        for step in range(2):
            opt.zero_grad()
            tokens = batches(step)
            loss = whole.loss(tokens[:, :-1], tokens[:, 1:])
            loss.backward()
            opt.step(1.0)
            want.append(float(loss))

        mesh = ParallelMesh(tp=1, fsdp=1, pp=world)
        torch.manual_seed(0)
        with torch.device(device):
            model = build_model(MODEL, VOCAB).to(dtype=torch.bfloat16)
        model.load_state_dict(state0)
        pipe = PipelineParallel(model, mesh.pp.group, 4)
        popt = FlatAdamW(pipe.module, 1e-3, (0.9, 0.95), 1e-8, 0.0, classes=pp_optimizer_classes(mesh.pp.group))
        got = []
        for step in range(2):
            popt.zero_grad()
            tokens = batches(step)
            got.append(float(pipe.loss(tokens[:, :-1], tokens[:, 1:])))
            popt.step(1.0)
        torch.cuda.synchronize()
        results[rank] = {"want": want, "got": got, "status": native.lib().ajb_check_status()}
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_pipeline_parallel_on_two_gpus():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, results)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    assert not alive, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs), [p.exitcode for p in procs]
    for rank in range(2):
        out = results[rank]
        assert out["status"] == 0, out
        for a, b in zip(out["got"], out["want"]):
            assert abs(a - b) < 3e-2 * max(1.0, abs(b)), out      # bf16 kernels, micro-batched sums
