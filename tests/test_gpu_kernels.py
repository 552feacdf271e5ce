"""Numerics of every sm_100a kernel against the plain PyTorch fp32 statement of the same op."""

import math

import pytest
import torch

from ajllm_b200 import ops
from ajllm_b200.ops import native, reference

pytestmark = pytest.mark.gpu


def _dev():
    return torch.device("cuda", 0)


def _rel_err(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.detach().float() - want.detach().float()).norm() / want.detach().float().norm().clamp_min(1e-12))


def test_native_library_is_loaded():
    assert native.available(), "the in-tree kernel library must be built before GPU tests run"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 512), (384, 1408, 2048), (1000, 520, 264),
                                    (4096, 4096, 2048), (130, 72, 4104)])
def test_gemm_forward_layout(m, n, k):
    torch.manual_seed(0)
    a = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(n, k, device=_dev(), dtype=torch.bfloat16)
    out = torch.empty(m, n, device=_dev(), dtype=torch.bfloat16)
    ops.gemm(a, b, out, m, n, k)
    want = a.float() @ b.float().t()
    assert _rel_err(out, want) < 5e-3


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (512, 2048, 1408), (1000, 264, 520), (2048, 2048, 4096)])
def test_gemm_dgrad_layout(m, n, k):
    """C[m,n] = A[m,k] @ B[k,n] with B stored [k,n] (n contiguous)."""
    torch.manual_seed(1)
    a = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(k, n, device=_dev(), dtype=torch.bfloat16)
    out = torch.empty(m, n, device=_dev(), dtype=torch.bfloat16)
    ops.gemm(a, b, out, m, n, k, b_mn_major=True)
    assert _rel_err(out, a.float() @ b.float()) < 5e-3


@pytest.mark.parametrize("m,n,k", [(256, 256, 128), (1408, 2048, 512), (264, 520, 1000), (2048, 2048, 8192)])
def test_gemm_wgrad_layout_accumulates_fp32(m, n, k):
    """C[m,n] += A^T B with A stored [k,m], B stored [k,n]; fp32 accumulation into C."""
    torch.manual_seed(2)
    a = torch.randn(k, m, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(k, n, device=_dev(), dtype=torch.bfloat16)
    acc = torch.randn(m, n, device=_dev(), dtype=torch.float32)
    want = acc + a.float().t() @ b.float()
    ops.gemm(a, b, acc, m, n, k, a_mn_major=True, b_mn_major=True, epilogue=1)
    assert _rel_err(acc, want) < 2e-3
    out = torch.empty(m, n, device=_dev(), dtype=torch.bfloat16)
    ops.gemm(a, b, out, m, n, k, a_mn_major=True, b_mn_major=True)
    assert _rel_err(out, a.float().t() @ b.float()) < 5e-3


@pytest.mark.parametrize("m,n,k", [(2048, 5632, 8192), (4096, 2048, 4096), (264, 520, 1000)])
def test_gemm_accumulate_with_k_slices(m, n, k):
    """Epilogue 3: C += A^T B where a long K may be cut into slices that add with reductions (352 or 256 tiles on
    148 SMs trigger the cut for the first two shapes; the third stays a single slice)."""
    torch.manual_seed(3)
    a = torch.randn(k, m, device=_dev(), dtype=torch.bfloat16)
    b = torch.randn(k, n, device=_dev(), dtype=torch.bfloat16)
    acc = torch.randn(m, n, device=_dev(), dtype=torch.float32)
    want = acc + a.float().t() @ b.float()
    ops.gemm(a, b, acc, m, n, k, a_mn_major=True, b_mn_major=True, epilogue=3)
    assert _rel_err(acc, want) < 2e-3


@pytest.mark.parametrize("a_mn,b_mn", [(False, False), (False, True), (True, True)])
@pytest.mark.parametrize("epilogue,split_k", [(0, 1), (1, 1), (2, 1), (3, 1), (3, 3)])
def test_gemm_on_cta_pairs(a_mn, b_mn, epilogue, split_k):
    """The cta_group::2 kernel on its own: ragged edges (rows 1152 = 4.5 pair tiles, columns 832, K 6208 = 97
    k-blocks) in every operand layout and epilogue, K slices included, against an fp32 matmul."""
    torch.manual_seed(5)
    m, n, k = 1152, 832, 6208
    a_rows = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    b_rows = torch.randn(n, k, device=_dev(), dtype=torch.bfloat16)
    a = a_rows.t().contiguous() if a_mn else a_rows
    b = b_rows.t().contiguous() if b_mn else b_rows
    want = a_rows.float() @ b_rows.float().t()
    if epilogue == 0:
        out = torch.zeros(m, n, device=_dev(), dtype=torch.bfloat16)
    else:
        out = torch.randn(m, n, device=_dev(), dtype=torch.float32)
        if epilogue in (1, 3):
            want = want + out
    native.call("ajb_gemm_bf16_pair", a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k, a.stride(0), b.stride(0),
                out.stride(0), int(a_mn), int(b_mn), epilogue, split_k, native.stream_ptr())
    torch.cuda.synchronize()
    assert native.lib().ajb_check_status() == 0
    assert _rel_err(out, want) < (5e-3 if epilogue == 0 else 2e-3)


def test_gemm_strided_operands():
    """Column slices of wider buffers are passed by leading dimension, not copied."""
    torch.manual_seed(3)
    wide = torch.randn(512, 1024, device=_dev(), dtype=torch.bfloat16)
    a = wide[:, 256:768]
    b = torch.randn(384, 512, device=_dev(), dtype=torch.bfloat16)
    outw = torch.zeros(512, 1024, device=_dev(), dtype=torch.bfloat16)
    ops.gemm(a, b, outw[:, 128:512], 512, 384, 512)
    assert _rel_err(outw[:, 128:512], a.float() @ b.float().t()) < 5e-3
    assert float(outw[:, :128].abs().max()) == 0.0 and float(outw[:, 512:].abs().max()) == 0.0


def test_linear_autograd_matches_reference():
    torch.manual_seed(4)
    x = torch.randn(4, 96, 512, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    w = (torch.randn(1024, 512, device=_dev()) * 0.05).to(torch.bfloat16).requires_grad_()
    y = ops.linear(x, w)
    g = torch.randn_like(y)
    y.backward(g)
    xr, wr = x.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    yr = reference.linear(xr, wr)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 5e-3 and _rel_err(x.grad, xr.grad) < 5e-3 and _rel_err(w.grad, wr.grad) < 5e-3


@pytest.mark.parametrize("rows,dim", [(300, 2048), (64, 4096), (17, 264), (5, 8192)])
def test_rmsnorm_with_residual(rows, dim):
    torch.manual_seed(5)
    x = torch.randn(rows, dim, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    d = torch.randn(rows, dim, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    g = (1 + 0.1 * torch.randn(dim, device=_dev())).to(torch.bfloat16).requires_grad_()
    h, y = ops.add_rms_norm(x, d, g, 1e-5)
    gh, gy = torch.randn_like(h), torch.randn_like(y)
    torch.autograd.backward([h, y], [gh, gy])
    xr, dr, gr = (t.detach().float().requires_grad_() for t in (x, d, g))
    hr = (xr + dr)
    # the kernel normalises the bf16-rounded residual stream
    hq = hr + (hr.detach().to(torch.bfloat16).float() - hr.detach())
    yr = reference.rms_norm(hq, gr, 1e-5)
    torch.autograd.backward([hr, yr], [gh.float(), gy.float()])
    assert _rel_err(h, hr) < 4e-3 and _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(d.grad, dr.grad) < 1e-2
    assert _rel_err(g.grad, gr.grad) < 2e-2


def test_swiglu_interleaved():
    torch.manual_seed(6)
    gu = torch.randn(257, 2 * 1408, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    act = ops.swiglu_interleaved(gu)
    g = torch.randn_like(act)
    act.backward(g)
    gur = gu.detach().float().requires_grad_()
    actr = reference.swiglu_interleaved(gur)
    actr.backward(g.float())
    assert _rel_err(act, actr) < 5e-3 and _rel_err(gu.grad, gur.grad) < 8e-3


@pytest.mark.parametrize("rows,d_model,d_ff", [(1024, 512, 1408), (777, 256, 352), (4096, 2048, 5632)])
def test_swiglu_inside_the_projection_epilogues(rows, d_model, d_ff):
    """The feed-forward block whose activation and activation gradient are computed by GEMM epilogues, against
    the fp32 statement and against the three-step path."""
    from ajllm_b200.ops import functional

    torch.manual_seed(60)
    dev = _dev()
    x = torch.randn(rows, d_model, device=dev, dtype=torch.bfloat16, requires_grad=True)
    w13 = (torch.randn(2 * d_ff, d_model, device=dev) * d_model ** -0.5).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(d_model, d_ff, device=dev) * d_ff ** -0.5).to(torch.bfloat16).requires_grad_()
    assert functional.FUSED_SWIGLU
    before = native.launch_count
    y = ops.swiglu_ffn(x, w13, w2)
    assert native.launch_count - before == 2        # two GEMMs, no separate activation kernel
    g = torch.randn_like(y)
    y.backward(g)
    xr, w13r, w2r = (t.detach().float().requires_grad_() for t in (x, w13, w2))
    yr = reference.linear(reference.swiglu_interleaved(reference.linear(xr, w13r)), w2r)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(w13.grad, w13r.grad) < 1e-2 and _rel_err(w2.grad, w2r.grad) < 1e-2
    # the same block as three steps (both round the pair to bf16 before the activation)
    x3, w133, w23 = (t.detach().clone().requires_grad_() for t in (x, w13, w2))
    y3 = ops.linear(ops.swiglu_interleaved(ops.linear(x3, w133)), w23)
    y3.backward(g)
    assert _rel_err(y3, y) < 1e-3
    assert _rel_err(x.grad, x3.grad) < 4e-3 and _rel_err(w13.grad, w133.grad) < 4e-3
    with torch.no_grad():
        assert _rel_err(ops.swiglu_ffn(x, w13, w2), y) < 1e-6     # inference form: the pre-activation is never written


def test_embedding_and_scatter_add():
    torch.manual_seed(7)
    table = torch.randn(1000, 256, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    ids = torch.randint(0, 1000, (4, 300), device=_dev())
    out = ops.embedding(ids, table)
    g = torch.randn_like(out)
    out.backward(g)
    tr = table.detach().float().requires_grad_()
    tr[ids].backward(g.float())
    assert torch.equal(out, table.detach()[ids])
    assert _rel_err(table.grad, tr.grad) < 5e-3


@pytest.mark.parametrize("rows,vocab", [(64, 32000), (33, 1000), (7, 8193)])
def test_cross_entropy_and_fused_head(rows, vocab):
    torch.manual_seed(8)
    dim = 256
    h = torch.randn(rows, dim, device=_dev(), dtype=torch.bfloat16, requires_grad=True)
    pad = (vocab + 7) // 8 * 8
    w = (torch.randn(pad, dim, device=_dev()) * 0.05).to(torch.bfloat16)[:vocab].requires_grad_()
    t = torch.randint(0, vocab, (rows,), device=_dev())
    loss = ops.linear_cross_entropy(h, w, t)
    loss.backward()
    hr, wr = h.detach().float().requires_grad_(), w.detach().float().requires_grad_()
    lr = reference.cross_entropy(reference.linear(hr, wr), t)
    lr.backward()
    assert abs(float(loss) - float(lr)) < 2e-2
    assert _rel_err(h.grad, hr.grad) < 3e-2 and _rel_err(w.grad, wr.grad) < 3e-2
    with torch.no_grad():
        assert abs(float(ops.linear_cross_entropy(h, w, t)) - float(lr)) < 2e-2


def test_sumsq_and_adamw_flat():
    from ajllm_b200.training.optim import flat_adamw, flat_sumsq

    torch.manual_seed(9)
    n = 1_000_003
    grad = torch.randn(n + 1, device=_dev())[:n]
    grad = grad.contiguous()
    ss = flat_sumsq(grad)
    assert abs(float(ss) - float(grad.double().square().sum())) / float(ss) < 1e-5
    assert float(flat_sumsq(grad)) == float(ss)          # fixed reduction order
    master = torch.randn(n, device=_dev())
    m, v = torch.zeros_like(master), torch.zeros_like(master)
    work = torch.empty(n, device=_dev(), dtype=torch.bfloat16)
    cm, cg, cmm, cv = master.cpu().clone(), grad.cpu().clone(), m.cpu().clone(), v.cpu().clone()
    for step in (1, 2):
        flat_adamw(master, grad, m, v, work, step, 1e-2, 0.9, 0.95, 1e-8, 0.1, ss, 1.0)
        flat_adamw(cm, cg, cmm, cv, None, step, 1e-2, 0.9, 0.95, 1e-8, 0.1, ss.cpu(), 1.0)
    assert float((master.cpu() - cm).abs().max()) < 1e-5
    assert torch.equal(work, master.to(torch.bfloat16))


@pytest.mark.parametrize("deterministic", [False, True])
@pytest.mark.parametrize("B,T,Hq,Hkv,hd", [(2, 256, 4, 2, 128), (1, 200, 2, 2, 128), (2, 384, 8, 2, 64), (1, 1024, 2, 1, 128),
                                           (2, 256, 16, 16, 32), (1, 200, 4, 2, 96)])
def test_flash_attention_forward_backward(B, T, Hq, Hkv, hd, deterministic, monkeypatch):
    """Both backward paths (fused single pass with reduced dQ; two reproducible kernels) against fp32 math."""
    from ajllm_b200.ops import functional
    monkeypatch.setattr(functional, "DETERMINISTIC_ATTENTION_BACKWARD", deterministic)
    torch.manual_seed(10)
    width = (Hq + 2 * Hkv) * hd
    qkv = (torch.randn(B, T, width, device=_dev()) * 0.5).to(torch.bfloat16).requires_grad_()
    cos, sin = reference.rope_tables(hd, T, 10000.0, device=_dev())
    ref_in = qkv.detach().float().requires_grad_()
    # the GPU path rotates q and k inside the packed buffer it is given, so hand it a copy
    out = ops.rope_attention(qkv.clone(), cos, sin, Hq, Hkv, hd)
    g = torch.randn_like(out)
    out.backward(g)

    q, k, v = ops.split_packed_qkv(ref_in, Hq, Hkv, hd)
    pos = torch.arange(T, device=_dev())
    qr, kr = reference.rope_interleaved(q, cos, sin, pos), reference.rope_interleaved(k, cos, sin, pos)
    want = reference.attention(qr, kr, v, causal=True).reshape(B, T, Hq * hd)
    want.backward(g.float())
    assert _rel_err(out, want) < 1.5e-2
    nq, nk = Hq * hd, Hkv * hd
    assert _rel_err(qkv.grad[..., :nq], ref_in.grad[..., :nq]) < 3e-2
    assert _rel_err(qkv.grad[..., nq:nq + nk], ref_in.grad[..., nq:nq + nk]) < 3e-2
    assert _rel_err(qkv.grad[..., nq + nk:], ref_in.grad[..., nq + nk:]) < 3e-2


def test_no_wait_expired():
    """Every bounded wait in the kernels above completed; a status word would mean a protocol bug."""
    assert native.lib().ajb_check_status() == 0


def test_batched_gemm_with_row_counts():
    torch.manual_seed(12)
    e, rows, k, n, seg = 3, 512, 256, 384, 256
    x = torch.randn(e, rows, k, device=_dev(), dtype=torch.bfloat16)
    w = (torch.randn(e, n, k, device=_dev()) * 0.1).to(torch.bfloat16)
    out = torch.empty(e, rows, n, device=_dev(), dtype=torch.bfloat16)
    ops.gemm_batched(x, w, out, rows, n, k)
    want = torch.einsum("erk,enk->ern", x.float(), w.float())
    assert _rel_err(out, want) < 5e-3
    counts = torch.tensor([[256, 100], [0, 129], [17, 0]], dtype=torch.int32, device=_dev())
    sentinel = torch.full_like(out, 7.0)
    ops.gemm_batched(x, w, sentinel, rows, n, k, valid_rows=counts, segment_rows=seg)
    for b in range(e):
        for s in range(2):
            c = int(counts[b, s])
            blocks = (c + 127) // 128 * 128
            got = sentinel[b, s * seg:(s + 1) * seg]
            assert _rel_err(got[:blocks], want[b, s * seg:s * seg + blocks]) < 5e-3 if blocks else True
            assert bool((got[blocks:] == 7.0).all())
    xg = x.clone().requires_grad_()
    wg = w.clone().requires_grad_()
    y = ops.linear_batched(xg, wg)
    g = torch.randn_like(y)
    y.backward(g)
    assert _rel_err(xg.grad, torch.einsum("ern,enk->erk", g.float(), w.float())) < 5e-3
    assert _rel_err(wg.grad, torch.einsum("ern,erk->enk", g.float(), x.float())) < 5e-3


@pytest.mark.parametrize("d_model,d_ff,with_counts", [(256, 352, False), (512, 1408, True), (256, 96, True)])
def test_stacked_swiglu_experts_in_the_batched_gemm_epilogues(d_model, d_ff, with_counts):
    """Per-expert SwiGLU blocks with the activation and its gradient inside the batched GEMMs, against fp32 math;
    with row counts, padding rows (zeros on the way in) stay zero and skipped row blocks are never touched."""
    torch.manual_seed(61)
    dev = _dev()
    e, rows, seg = 3, 512, 256
    counts = torch.tensor([[256, 100], [0, 129], [17, 0]], dtype=torch.int32, device=dev) if with_counts else None
    x = torch.randn(e, rows, d_model, device=dev, dtype=torch.bfloat16)
    g = torch.randn(e, rows, d_model, device=dev, dtype=torch.bfloat16)
    if with_counts:
        keep = torch.zeros(e, rows, 1, device=dev, dtype=torch.bool)
        for b in range(e):
            for s in range(2):
                keep[b, s * seg:s * seg + int(counts[b, s])] = True
        x, g = x * keep, g * keep          # the dispatch buffer holds zeros behind the rows in use
    x.requires_grad_()
    w13 = (torch.randn(e, 2 * d_ff, d_model, device=dev) * d_model ** -0.5).to(torch.bfloat16).requires_grad_()
    w2 = (torch.randn(e, d_model, d_ff, device=dev) * d_ff ** -0.5).to(torch.bfloat16).requires_grad_()
    before = native.launch_count
    y = ops.swiglu_ffn_batched(x, w13, w2, counts, seg if with_counts else 0)
    assert native.launch_count - before == 2
    y.backward(g)
    xr, w13r, w2r = (t.detach().float().requires_grad_() for t in (x, w13, w2))
    hidden = reference.swiglu_interleaved(torch.einsum("erk,enk->ern", xr, w13r))
    yr = torch.einsum("erf,edf->erd", hidden, w2r)
    yr.backward(g.float())
    assert _rel_err(y, yr) < 8e-3
    assert _rel_err(x.grad, xr.grad) < 1e-2 and _rel_err(w13.grad, w13r.grad) < 1e-2 and _rel_err(w2.grad, w2r.grad) < 1e-2
    if with_counts:
        assert float(y[~keep.expand_as(y)].abs().max()) == 0.0


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (16, 6144, 4096), (64, 4096, 14336), (128, 4096, 4096),
                                   (37, 1000, 4104), (128, 6144, 520)])
def test_decoding_gemm_with_cluster_reduction(m, n, k):
    """Few rows, few 128-row weight strips: one cluster of CTAs per strip, K slices summed through distributed shared
    memory (ragged n and k included), against an fp32 matmul; called twice in a row."""
    from ajllm_b200.ops.functional import _linear_decode

    torch.manual_seed(19)
    x = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    w = (torch.randn(n, k, device=_dev()) * 0.05).to(torch.bfloat16)
    with torch.no_grad():
        for _ in range(2):
            got = _linear_decode(x, w)
    torch.cuda.synchronize()
    assert native.lib().ajb_check_status() == 0
    assert _rel_err(got, x.float() @ w.float().t()) < 5e-3


@pytest.mark.parametrize("m,n,k", [(1, 4096, 4096), (128, 6144, 4096), (256, 4096, 14336), (40, 1000, 264),
                                   (256, 6144, 4096), (200, 28672, 4096), (384, 1000, 512), (512, 4096, 4096)])
def test_split_k_linear_for_few_rows(m, n, k):
    from ajllm_b200.ops.functional import linear_skinny

    torch.manual_seed(13)
    x = torch.randn(m, k, device=_dev(), dtype=torch.bfloat16)
    w = (torch.randn(n, k, device=_dev()) * 0.05).to(torch.bfloat16)
    got = linear_skinny(x, w)
    assert _rel_err(got, x.float() @ w.float().t()) < 5e-3
    with torch.no_grad():
        assert _rel_err(ops.linear(x, w), x.float() @ w.float().t()) < 5e-3
