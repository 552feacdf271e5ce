"""The multi-GPU kernels on ONE GPU: rank 0 of a 2 / 4 / 8-rank group whose peer buffers are tensors on the same
device and whose handshake words are preset, so that every mode, tile variant and the double-buffered call protocol
of ``csrc/comm_gemm.cu`` and the dispatch / combine kernels of ``csrc/moe.cu`` are checked against fp32 math wherever
the GPU tests run. The same kernels run over real NVLink peers in ``test_gpu_fused_tp.py`` / ``test_gpu_moe.py``."""

import ctypes

import pytest
import torch

from ajllm_b200.ops import native

pytestmark = pytest.mark.gpu

BF = torch.bfloat16


def _rel(got, want):
    return float((got.float() - want.float()).norm() / want.float().norm().clamp_min(1e-12))


def _group(tp):
    from ajllm_b200.parallel.emulated_group import EmulatedGroup
    return EmulatedGroup(torch.device("cuda", 0), tp)


# m_local 256 / 512: CTA pairs (256-row tiles); 128 / 384: single CTAs. n 1000 leaves a ragged last column tile.
@pytest.mark.parametrize("tp,m_local,n,k,b_mn", [(2, 512, 1024, 512, False), (2, 384, 1000, 256, False),
                                                 (4, 256, 768, 512, True), (8, 128, 512, 384, False),
                                                 (8, 256, 1000, 256, True)])
def test_all_gather_gemm_as_rank_0(tp, m_local, n, k, b_mn):
    from ajllm_b200.parallel.emulated_group import MODE_ALL_GATHER
    dev = torch.device("cuda", 0)
    torch.manual_seed(tp * 1000 + m_local)
    group = _group(tp)
    m = tp * m_local
    x = (torch.randn(m, k, device=dev) * 0.5).to(BF)
    w = (torch.randn(n, k, device=dev) * 0.1).to(BF)
    weight = w.t().contiguous() if b_mn else w          # stored [k, n] when n-major
    stage = [x[r * m_local:(r + 1) * m_local].contiguous() for r in range(tp)]
    want = x.float() @ w.float().t()
    for call in range(4):                               # four calls: epochs advance, flags of earlier calls stay behind
        gathered = torch.zeros(m, k, device=dev, dtype=BF)
        gathered[:m_local].copy_(stage[0])
        out = torch.zeros(m, n, device=dev, dtype=BF)
        # the last call asks for more pulling CTAs than its SM budget holds: the launch keeps half of it for the products
        group.copy_ctas = 96 if call == 3 else 20
        group.launch(MODE_ALL_GATHER, m, n, k, out, b=weight, b_mn=b_mn, gathered=gathered, stage=stage,
                     sm_budget=64 if call == 2 else (40 if call == 3 else None))
        torch.cuda.synchronize()
        assert torch.equal(gathered, x)
        assert _rel(out, want) < 5e-3, (call, _rel(out, want))
    assert native.check_status() == 0


@pytest.mark.parametrize("tp,m_local,d_model,d_ff", [(2, 512, 512, 704), (4, 256, 256, 352), (8, 128, 256, 1408), (2, 384, 384, 96)])
def test_swiglu_epilogues_of_the_all_gather_gemm_as_rank_0(tp, m_local, d_model, d_ff):
    """Forward: gathered x @ w13^T leaves (gate, up) pairs and the activation from one kernel. Backward: gathered
    d_out @ w2 leaves the gradient of the pairs; d_act is never stored."""
    from ajllm_b200.ops import reference
    from ajllm_b200.parallel.emulated_group import MODE_ALL_GATHER
    dev = torch.device("cuda", 0)
    torch.manual_seed(tp * 31 + d_ff)
    group = _group(tp)
    m = tp * m_local
    x = (torch.randn(m, d_model, device=dev) * 0.5).to(BF)
    w13 = (torch.randn(2 * d_ff, d_model, device=dev) * d_model ** -0.5).to(BF)
    w2 = (torch.randn(d_model, d_ff, device=dev) * d_ff ** -0.5).to(BF)
    # forward
    stage = [x[r * m_local:(r + 1) * m_local].contiguous() for r in range(tp)]
    gathered = torch.zeros(m, d_model, device=dev, dtype=BF)
    gathered[:m_local].copy_(stage[0])
    gate_up = torch.zeros(m, 2 * d_ff, device=dev, dtype=BF)
    act = torch.zeros(m, d_ff, device=dev, dtype=BF)
    group.launch(MODE_ALL_GATHER, m, 2 * d_ff, d_model, gate_up, b=w13, gathered=gathered, stage=stage, swiglu=1, aux=act)
    torch.cuda.synchronize()
    assert _rel(gate_up, x.float() @ w13.float().t()) < 5e-3
    assert _rel(act, reference.swiglu_interleaved(gate_up.float())) < 4e-3        # from the bf16-rounded pairs
    # backward
    d_out = (torch.randn(m, d_model, device=dev)).to(BF)
    stage = [d_out[r * m_local:(r + 1) * m_local].contiguous() for r in range(tp)]
    gathered = torch.zeros(m, d_model, device=dev, dtype=BF)
    gathered[:m_local].copy_(stage[0])
    d_gate_up = torch.zeros(m, 2 * d_ff, device=dev, dtype=BF)
    group.launch(MODE_ALL_GATHER, m, d_ff, d_model, d_gate_up, b=w2, b_mn=True, gathered=gathered, stage=stage,
                 swiglu=2, aux=gate_up)
    torch.cuda.synchronize()
    pairs = gate_up.float().requires_grad_()
    reference.swiglu_interleaved(pairs).backward(d_out.float() @ w2.float())
    assert torch.equal(gathered, d_out)
    assert _rel(d_gate_up, pairs.grad) < 6e-3
    assert native.check_status() == 0


@pytest.mark.parametrize("tp,m_local,n,k,b_mn", [(2, 512, 1024, 512, False), (2, 128, 1000, 256, True),
                                                 (4, 256, 512, 256, False), (8, 256, 768, 128, False),
                                                 (8, 384, 256, 256, True)])
def test_gemm_reduce_scatter_as_rank_0_alternates_its_receive_buffers(tp, m_local, n, k, b_mn):
    from ajllm_b200.parallel.emulated_group import MODE_REDUCE_SCATTER
    dev = torch.device("cuda", 0)
    torch.manual_seed(tp * 77 + n)
    group = _group(tp)
    m = tp * m_local
    x = (torch.randn(m, k, device=dev) * 0.5).to(BF)
    w = (torch.randn(n, k, device=dev) * 0.1).to(BF)
    weight = w.t().contiguous() if b_mn else w
    own = x.float() @ w.float().t()                     # this rank's partial product for every row
    # two sets of receive buffers (odd / even calls); the peers' partial sums for rank 0's rows differ per set
    sets = []
    for parity in (0, 1):
        recv = [torch.zeros(tp, m_local, n, device=dev, dtype=BF) for _ in range(tp)]
        for r in range(1, tp):
            recv[0][r].copy_((torch.randn(m_local, n, device=dev) * (1 + parity)).to(BF))
        sets.append(recv)
    tiles = (m_local // 128) * ((n + 255) // 256)
    for call in range(1, 5):
        out = torch.zeros(m_local, n, device=dev, dtype=BF)
        parity = group.receive_parity()
        assert parity == call & 1
        group.launch(MODE_REDUCE_SCATTER, m, n, k, out, b=weight, b_mn=b_mn, a=x, recv=sets[1], recv_even=sets[0],
                     tiles_for_count=tiles, sm_budget=48 if call == 4 else None)
        torch.cuda.synchronize()
        want = own[:m_local] + sum(sets[parity][0][r].float() for r in range(1, tp))
        assert _rel(out, want) < 5e-3, (call, _rel(out, want))
        # the partial tiles for the other ranks' rows landed in THEIR buffers of this parity, slot 0
        for r in range(1, tp):
            assert _rel(sets[parity][r][0], own[r * m_local:(r + 1) * m_local]) < 5e-3
    assert [int(v) for v in group.reduce_state[:2].tolist()] == [4, group.expected]
    assert native.check_status() == 0


@pytest.mark.parametrize("rows", [16, 128, 200])
def test_gemm_all_reduce_as_rank_0(rows):
    from ajllm_b200.parallel.emulated_group import MODE_ALL_REDUCE
    dev = torch.device("cuda", 0)
    torch.manual_seed(rows)
    group = _group(2)
    n, k = 1024, 512
    m = -(-rows // 128) * 128
    x = (torch.randn(rows, k, device=dev) * 0.5).to(BF)
    w = (torch.randn(n, k, device=dev) * 0.1).to(BF)
    peer = (torch.randn(m, n, device=dev)).to(BF)
    recv = [torch.zeros(2, m, n, device=dev, dtype=BF) for _ in range(2)]
    recv[0][1].copy_(peer)
    tiles = (m // 128) * ((n + 255) // 256)
    for _ in range(3):                                   # the same buffers serve both parities here
        out = torch.zeros(m, n, device=dev, dtype=BF)
        group.launch(MODE_ALL_REDUCE, m, n, k, out, b=w, a=x, recv=recv, tiles_for_count=tiles, a_rows=rows)
        torch.cuda.synchronize()
        want = x.float() @ w.float().t() + peer[:rows].float()
        assert _rel(out[:rows], want) < 5e-3
    assert native.check_status() == 0


def test_gather_weight_gemm_as_rank_0():
    from ajllm_b200.parallel.emulated_group import MODE_GATHER_WEIGHT
    dev = torch.device("cuda", 0)
    torch.manual_seed(5)
    group = _group(2)
    m, n, k, offset = 512, 768, 512, 4096
    x = (torch.randn(m, k, device=dev) * 0.5).to(BF)
    w = (torch.randn(n, k, device=dev) * 0.1).to(BF)
    shard = (offset + n * k + 4096 + 15) // 16 * 8
    flat_all = torch.zeros(2 * shard, device=dev, dtype=BF)
    flat_all[offset:offset + n * k].copy_(w.reshape(-1))
    stage = [flat_all[:shard].contiguous(), flat_all[shard:].contiguous()]
    for _ in range(2):
        flat = torch.zeros(2 * shard, device=dev, dtype=BF)
        flat[:shard].copy_(stage[0])
        out = torch.zeros(m, n, device=dev, dtype=BF)
        group.launch(MODE_GATHER_WEIGHT, m, n, k, out, b=flat, a=x, gathered=flat, stage=stage, shard_elems=shard,
                     b_offset=offset)
        torch.cuda.synchronize()
        assert torch.equal(flat, flat_all)
        assert _rel(out, x.float() @ w.float().t()) < 5e-3
    assert native.check_status() == 0


# ------------------------------------------------------------------------------------------ expert exchange
def _exchange_args(ep, tokens, top_k, dim, local_experts, stride, slots, buffers, flags, counts_sym, counts, epoch, local):
    from ajllm_b200.parallel.moe_exchange import _Args
    a = _Args()
    a.tokens, a.top_k, a.dim, a.ep, a.rank = tokens, top_k, dim, ep, 0
    a.local_experts, a.stride = local_experts, stride
    a.slots = slots.data_ptr()
    for r in range(ep):
        a.peer_buffers[r] = buffers[r].data_ptr()
        a.flag_ptrs[r] = flags[r].data_ptr()
        a.peer_counts[r] = counts_sym[r].data_ptr()
    a.counts = counts.data_ptr() if counts is not None else None
    a.epoch = epoch
    a.local_counter = local.data_ptr()
    return a


@pytest.mark.parametrize("ep", [2, 4, 8])
def test_expert_dispatch_and_combine_as_rank_0(ep):
    dev = torch.device("cuda", 0)
    torch.manual_seed(ep)
    lib = native.lib()
    from ajllm_b200.parallel.moe_exchange import _Args
    push, pull = lib.ajb_moe_push_rows, lib.ajb_moe_pull_rows
    push.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    pull.argtypes = [ctypes.POINTER(_Args), ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    push.restype = pull.restype = ctypes.c_int
    tokens, top_k, dim, local_experts, stride = 300, 3, 264, 2, 256
    experts = ep * local_experts
    # distinct (expert, position) slots per assignment; about a tenth dropped (-1)
    choice = torch.stack([torch.randperm(experts, device=dev)[:top_k] for _ in range(tokens)])
    position = torch.zeros(tokens, top_k, dtype=torch.long, device=dev)
    fill = [0] * experts
    for t in range(tokens):
        for j in range(top_k):
            e = int(choice[t, j])
            position[t, j] = fill[e]
            fill[e] += 1
    assert max(fill) <= stride
    slots = (choice * stride + position).to(torch.int32)
    slots[torch.rand(tokens, top_k, device=dev) < 0.1] = -1
    rows = torch.randn(tokens, dim, device=dev).to(BF)
    scale = torch.rand(tokens, top_k, device=dev) + 0.5
    buffers = [torch.zeros(local_experts * ep * stride, dim, device=dev, dtype=BF) for _ in range(ep)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(ep)]
    counts_sym = [torch.zeros(4096, dtype=torch.int32, device=dev) for _ in range(ep)]
    counts = torch.tensor(fill, dtype=torch.int32, device=dev)
    local = torch.zeros(4, dtype=torch.int32, device=dev)

    def dest(slot):
        e, pos = divmod(slot, stride)
        r, le = divmod(e, local_experts)
        return r, (le * ep + 0) * stride + pos

    for epoch, use_scale in ((1, False), (2, True)):
        for b in buffers:
            b.zero_()
        flags[0][0:ep] = epoch              # every peer's "my rows have arrived" word for this call
        args = _exchange_args(ep, tokens, top_k, dim, local_experts, stride, slots, buffers, flags, counts_sym, counts, epoch, local)
        assert push(ctypes.byref(args), rows.data_ptr(), scale.data_ptr() if use_scale else None, native.stream_ptr()) == 0
        torch.cuda.synchronize()
        want = [torch.zeros_like(b) for b in buffers]
        host_slots = slots.cpu()
        for t in range(tokens):
            for j in range(top_k):
                s = int(host_slots[t, j])
                if s < 0:
                    continue
                r, row = dest(s)
                want[r][row] = (rows[t].float() * (scale[t, j] if use_scale else 1.0)).to(BF)
        for r in range(ep):
            assert torch.equal(buffers[r], want[r]), (epoch, r)
        for r in range(ep):                 # kept-row counts per (local expert, source rank 0)
            got = counts_sym[r][:local_experts * ep].view(local_experts, ep)[:, 0]
            assert got.tolist() == fill[r * local_experts:(r + 1) * local_experts]

    # combine: every rank's buffer holds expert outputs; out[t] = sum_j w[t, j] * row(t, j), dots[t, j] = <up[t], row(t, j)>
    for b in buffers:
        b.copy_(torch.randn_like(b, dtype=torch.float32).to(BF))
    weights = torch.rand(tokens, top_k, device=dev)
    upstream = torch.randn(tokens, dim, device=dev).to(BF)
    epoch = 3
    flags[0][8:8 + ep] = epoch              # release words
    flags[0][16:16 + ep] = epoch            # the peers' buffers are ready for this call
    out = torch.zeros(tokens, dim, device=dev, dtype=BF)
    dots = torch.zeros(tokens, top_k, device=dev)
    args = _exchange_args(ep, tokens, top_k, dim, local_experts, stride, slots, buffers, flags, counts_sym, None, epoch, local)
    assert pull(ctypes.byref(args), out.data_ptr(), weights.data_ptr(), upstream.data_ptr(), dots.data_ptr(), native.stream_ptr()) == 0
    torch.cuda.synchronize()
    want_out = torch.zeros(tokens, dim, device=dev)
    want_dots = torch.zeros(tokens, top_k, device=dev)
    host_slots = slots.cpu()
    for t in range(tokens):
        for j in range(top_k):
            s = int(host_slots[t, j])
            if s < 0:
                continue
            r, row = dest(s)
            src = buffers[r][row].float()
            want_out[t] += weights[t, j] * src
            want_dots[t, j] = (upstream[t].float() * src).sum()
    assert _rel(out, want_out) < 5e-3
    assert _rel(dots, want_dots) < 1e-3
    assert native.check_status() == 0
