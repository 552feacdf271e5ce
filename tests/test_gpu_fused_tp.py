"""Fused all-gather->GEMM and GEMM->reduce-scatter kernels against the NCCL + GEMM composition and an
fp32 reference, on 2 GPUs (skipped where fewer are visible). Ranks are child processes, one per GPU."""

import os

import pytest
import torch

from tests.conftest import free_port

pytestmark = pytest.mark.gpu


def _worker(rank: int, world: int, port: int, rows_local: int, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from ajllm_b200 import ops
        from ajllm_b200.ops import native
        from ajllm_b200.parallel.fused import FusedTensorParallel
        from ajllm_b200.parallel.tensor_parallel import TensorParallel

        fused = FusedTensorParallel(dist.group.WORLD, device)
        plain = TensorParallel(dist.group.WORLD, rank, world)
        with_fused = TensorParallel(dist.group.WORLD, rank, world, fused=fused)
        d_model, n_local = 512, 384

        def rel(a, b):
            return float((a.float() - b.float()).norm() / b.float().norm().clamp_min(1e-12))

        errors = {}
        for trial in range(2):          # twice: buffers, flags and counters are reused across calls
            torch.manual_seed(100 + trial)       # same seed on every rank: full tensors are known everywhere
            x_full = (torch.randn(rows_local * world, d_model, device=device) * 0.5).to(torch.bfloat16)
            w_col = (torch.randn(world, n_local, d_model, device=device) * 0.05).to(torch.bfloat16)
            w_row = (torch.randn(world, d_model, n_local, device=device) * 0.05).to(torch.bfloat16)
            g_col = torch.randn(rows_local * world, n_local, device=device).to(torch.bfloat16)
            g_row = torch.randn(rows_local * world, d_model, device=device).to(torch.bfloat16)
            for tp, tag in ((with_fused, "fused"), (plain, "nccl")):
                x = x_full[rank * rows_local:(rank + 1) * rows_local].clone().requires_grad_()
                w = w_col[rank].clone().requires_grad_()
                y = tp.gather_linear(x, w)
                y.backward(g_col)
                want_y = x_full.float() @ w_col[rank].float().t()
                want_dx = sum(g_col.float() @ w_col[r].float() for r in [rank])   # this rank's partial only
                errors[f"{tag}/ag/y/{trial}"] = rel(y, want_y)
                errors[f"{tag}/ag/dw/{trial}"] = rel(w.grad, g_col.float().t() @ x_full.float())
                # dx is the sum over ranks of dY_r W_r restricted to this rank's rows; every rank used the same dY here
                total = torch.zeros(rows_local * world, d_model, device=device)
                for r in range(world):
                    total += g_col.float() @ w_col[r].float()
                errors[f"{tag}/ag/dx/{trial}"] = rel(x.grad, total[rank * rows_local:(rank + 1) * rows_local])

                a = (x_full[:, :n_local] * (rank + 1)).contiguous().requires_grad_()
                wr = w_row[rank].clone().requires_grad_()
                z = tp.linear_scatter(a, wr)
                z.backward(g_row[rank * rows_local:(rank + 1) * rows_local])
                want_z = torch.zeros(rows_local * world, d_model, device=device)
                for r in range(world):
                    want_z += (x_full[:, :n_local].float() * (r + 1)) @ w_row[r].float().t()
                errors[f"{tag}/rs/z/{trial}"] = rel(z, want_z[rank * rows_local:(rank + 1) * rows_local])
                errors[f"{tag}/rs/da/{trial}"] = rel(a.grad, g_row.float() @ w_row[rank].float())
                errors[f"{tag}/rs/dw/{trial}"] = rel(wr.grad, g_row.float().t() @ (x_full[:, :n_local].float() * (rank + 1)))
        # the same call twice must give the same bits (a race in the flag / epoch protocol would show here), and
        # nobody may have written behind the end of a symmetric buffer
        torch.manual_seed(9)
        xs = (torch.randn(rows_local, d_model, device=device) * 0.5).to(torch.bfloat16)
        ws = (torch.randn(n_local, d_model, device=device) * 0.05).to(torch.bfloat16)
        first = [fused.all_gather_gemm(xs, ws, False, n_local, d_model)[1].clone() for _ in range(2)]
        errors["repeat/ag"] = 0.0 if torch.equal(first[0], first[1]) else 1.0
        # the kernel also leaves every rank's rows (its own included) in the gathered activations
        got_rows = fused.all_gather_gemm(xs, ws, False, n_local, d_model)[0]
        want_rows = torch.empty_like(got_rows)
        dist.all_gather_into_tensor(want_rows, xs)
        errors["ag/gathered"] = 0.0 if torch.equal(got_rows, want_rows) else 1.0
        xa = (torch.randn(rows_local * world, n_local, device=device) * 0.5).to(torch.bfloat16)
        wr = (torch.randn(d_model, n_local, device=device) * 0.05).to(torch.bfloat16)
        second = [fused.gemm_reduce_scatter(xa, wr, False, d_model, n_local).clone() for _ in range(2)]
        errors["repeat/rs"] = 0.0 if torch.equal(second[0], second[1]) else 1.0
        errors["guards"] = 0.0 if fused.guards_intact() else 1.0
        torch.cuda.synchronize()
        status = native.lib().ajb_check_status()
        results[rank] = {"errors": errors, "status": status}
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("rows_local", [128, 1024])
def test_fused_tensor_parallel_kernels_match_nccl_path(rows_local):
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, rows_local, results)) for r in range(2)]
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
        bad = {k: v for k, v in out["errors"].items() if not v < 2e-2}
        assert not bad, bad


def _all_reduce_worker(rank: int, world: int, port: int, results):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    device = torch.device("cuda", rank)
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=device)
    try:
        from ajllm_b200.ops import native
        from ajllm_b200.parallel.fused import FusedTensorParallel

        fused = FusedTensorParallel(dist.group.WORLD, device)
        errors = {}
        # decoding shapes: a handful of rows up to a few hundred, K sharded over the ranks; interleaved with a
        # reduce-scatter call because both modes share receive buffer, counters and handshake words
        for trial, (rows, n, k_local) in enumerate([(5, 512, 256), (128, 1024, 384), (300, 768, 512), (5, 512, 256)]):
            torch.manual_seed(7 + trial)
            x_all = (torch.randn(world, rows, k_local, device=device) * 0.5).to(torch.bfloat16)
            w_all = (torch.randn(world, n, k_local, device=device) * 0.05).to(torch.bfloat16)
            got = fused.gemm_all_reduce(x_all[rank].contiguous(), w_all[rank].contiguous())
            want = sum(x_all[r].float() @ w_all[r].float().t() for r in range(world))
            errors[f"ar/{trial}"] = float((got.float() - want).norm() / want.norm())
            if trial == 1:
                a = (torch.randn(256, k_local, device=device) * 0.5).to(torch.bfloat16)
                fused.gemm_reduce_scatter(a, w_all[rank].contiguous(), False, n, k_local)
        # fully sharded weights: W [n, k] sits at an offset inside a flat buffer whose equal slices (cut in the
        # middle of a row) live on the ranks; the slices are gathered while x @ W^T is computed
        for trial, (rows, n, k, offset, shard) in enumerate([(256, 640, 512, 0, 170000), (128, 304, 256, 4096, 64008)]):
            torch.manual_seed(31 + trial)
            flat_all = (torch.randn(world * shard, device=device) * 0.05).to(torch.bfloat16)
            x = (torch.randn(rows, k, device=device) * 0.5).to(torch.bfloat16)
            flat, got = fused.gather_weight_gemm(x, flat_all[rank * shard:(rank + 1) * shard].clone(), n, k, offset)
            w = flat_all[offset:offset + n * k].view(n, k)
            want = x.float() @ w.float().t()
            errors[f"gw/{trial}"] = float((got.float() - want).norm() / want.norm())
            errors[f"gw/flat/{trial}"] = float((flat.float() - flat_all.float()).abs().max())
        torch.cuda.synchronize()
        results[rank] = {"errors": errors, "status": native.lib().ajb_check_status()}
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_fused_gemm_all_reduce_for_decoding():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    manager = ctx.Manager()
    results = manager.dict()
    port = free_port()
    procs = [ctx.Process(target=_all_reduce_worker, args=(r, 2, port, results)) for r in range(2)]
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
        bad = {k: v for k, v in out["errors"].items() if not v < 2e-2}
        assert not bad, bad
