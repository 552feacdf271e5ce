"""Differentiable ops. CPU tensors run the oracle math in :mod:`ajllm_b200.ops.reference` under
autograd; CUDA tensors run the sm_100a kernels through hand-written backward passes.

GPU data layout: activations are bf16 ``[tokens, features]`` row-major; the three attention
projections are one GEMM whose output row is ``[q heads | k heads | v heads]`` and the attention
kernels read that packed row in place; the two SwiGLU input projections are one GEMM whose output
interleaves gate (even) and up (odd) columns so the activation pairs sit side by side.
"""

from __future__ import annotations

import contextlib
import math
import os

import torch

from ajllm_b200.ops import native, reference

EPI_STORE_BF16 = 0
EPI_ACCUM_F32 = 1
EPI_STORE_F32 = 2
EPI_ADD_F32 = 3         # accumulate; long-K products may be cut into K slices that add with reductions (order not fixed)


def wgrad_epilogue() -> int:
    """Epilogue of a weight-gradient GEMM that accumulates into ``main_grad``."""
    return EPI_ACCUM_F32 if DETERMINISTIC_WGRAD else EPI_ADD_F32

# Attention backward: False selects the fused single-pass kernel (dQ summed with fp32 reductions, last
# bits may differ between runs); True (or AJB_DETERMINISTIC_ATTENTION=1) the bit-reproducible two-kernel path.
DETERMINISTIC_ATTENTION_BACKWARD = os.environ.get("AJB_DETERMINISTIC_ATTENTION", os.environ.get("AJB_DETERMINISTIC", "0")) == "1"
# Weight gradients accumulated into ``main_grad``: with AJB_DETERMINISTIC=1 every output tile is owned by one CTA.
DETERMINISTIC_WGRAD = os.environ.get("AJB_DETERMINISTIC", "0") == "1"


def _is_cuda(t: torch.Tensor) -> bool:
    return t.device.type == "cuda"


# CUDA tensors run the kernels of this package, which compute in bf16 (fp32 lives in the optimizer's master weights,
# gradients and moments). Another dtype on a GPU is an error rather than a silent drop to eager PyTorch; a caller that
# wants eager math on purpose (the `baseline` arm of the acceleration benchmark) says so with `eager_cuda()`.
_EAGER_CUDA_ALLOWED = False


@contextlib.contextmanager
def eager_cuda():
    """Inside this block non-bf16 CUDA tensors take the plain PyTorch math of :mod:`ajllm_b200.ops.reference`."""
    global _EAGER_CUDA_ALLOWED
    previous, _EAGER_CUDA_ALLOWED = _EAGER_CUDA_ALLOWED, True
    try:
        yield
    finally:
        _EAGER_CUDA_ALLOWED = previous


def _native(t: torch.Tensor, op: str) -> bool:
    """True when ``t`` goes to the CUDA kernels; False for the oracle math (CPU tensors, or eager CUDA on request)."""
    if t.device.type != "cuda":
        return False
    if t.dtype == torch.bfloat16:
        return True
    if _EAGER_CUDA_ALLOWED:
        return False
    raise TypeError(f"{op}: CUDA tensors must be bfloat16 (got {t.dtype}); cast the model with .to(torch.bfloat16) - "
                    "fp32 master weights are kept by the optimizer - or wrap the call in ops.eager_cuda()")


# ----------------------------------------------------------------------------- weight-gradient stream

# Weight-gradient GEMMs accumulate into the optimizer's fp32 buffer and nothing in the backward pass reads their
# result, so they need not sit on the critical path: with a side stream set, each one is issued there (ordered after
# the kernels that produced its operands) and runs beside whatever the main stream does next - in particular beside
# a tensor-parallel projection that is waiting on NVLink with most SMs idle. All of them share the one stream, so
# the read-modify-write accumulations into one buffer stay serialised even when several micro-batches are in flight.
_WGRAD_STREAM: "torch.cuda.Stream | None" = None


def set_wgrad_stream(stream) -> None:
    global _WGRAD_STREAM
    _WGRAD_STREAM = stream


def wgrad_stream():
    return _WGRAD_STREAM


def join_wgrad_stream() -> None:
    """The current stream waits for every weight gradient issued so far (call before the optimizer reads them)."""
    if _WGRAD_STREAM is not None:
        torch.cuda.current_stream().wait_stream(_WGRAD_STREAM)


def wgrad_accumulate(grad_out: torch.Tensor, activations: torch.Tensor, main_grad: torch.Tensor, n: int, k: int,
                     m: int) -> None:
    """``main_grad[n, k] += grad_out[m, n]^T @ activations[m, k]`` (fp32 accumulation in place)."""
    side = _WGRAD_STREAM
    if side is None or not grad_out.is_cuda:
        gemm(grad_out, activations, main_grad, n, k, m, a_mn_major=True, b_mn_major=True, epilogue=wgrad_epilogue())
        return
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        gemm(grad_out, activations, main_grad, n, k, m, a_mn_major=True, b_mn_major=True, epilogue=wgrad_epilogue())
    # the operands were allocated on the producing stream: keep their memory out of reuse until the side stream is done
    grad_out.record_stream(side)
    activations.record_stream(side)


# ----------------------------------------------------------------------------- GEMM


def gemm(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, m: int, n: int, k: int, *,
         a_mn_major: bool = False, b_mn_major: bool = False, epilogue: int = EPI_STORE_BF16) -> torch.Tensor:
    """``out[m,n] (+)= op(a)[m,k] @ op(b)[k,n]`` on the tcgen05 kernel.

    ``a`` is stored ``[m,k]`` (k contiguous) or, with ``a_mn_major``, ``[k,m]`` (m contiguous); ``b`` is
    stored ``[n,k]`` (k contiguous) or, with ``b_mn_major``, ``[k,n]`` (n contiguous). Leading dimensions
    come from ``stride(0)`` so column slices of wider buffers can be passed without a copy.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    native.call("ajb_gemm_bf16", a.data_ptr(), b.data_ptr(), out.data_ptr(), m, n, k,
                a.stride(0), b.stride(0), out.stride(0), int(a_mn_major), int(b_mn_major), epilogue,
                native.stream_ptr())
    return out


def gemm_batched(a: torch.Tensor, b: torch.Tensor, out: torch.Tensor, m: int, n: int, k: int, *,
                 a_mn_major: bool = False, b_mn_major: bool = False, epilogue: int = EPI_STORE_BF16,
                 valid_rows: torch.Tensor | None = None, segment_rows: int = 0) -> torch.Tensor:
    """``batch`` equal-shaped GEMMs in one launch: ``a``, ``b``, ``out`` are 3-D with the problem index first.
    ``valid_rows`` (int32 ``[batch, m / segment_rows]`` on the device) marks how many leading rows of each row
    segment hold data; row blocks past that are skipped and their outputs left untouched."""
    batch = a.shape[0]
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and out.stride(-1) == 1
    native.call("ajb_gemm_bf16_batched", a.data_ptr(), b.data_ptr(), out.data_ptr(), batch, m, n, k,
                a.stride(1), b.stride(1), out.stride(1), a.stride(0), b.stride(0), out.stride(0),
                int(a_mn_major), int(b_mn_major), epilogue, native.ptr(valid_rows), segment_rows, native.stream_ptr())
    return out


class _BatchedLinearFn(torch.autograd.Function):
    """``y[e] = x[e] @ w[e].T`` for stacked experts, with optional per-segment row counts."""

    @staticmethod
    def forward(ctx, x, weight, valid_rows, segment_rows):
        e, rows, k = x.shape
        n = weight.shape[1]
        x = x.contiguous()
        out = torch.zeros(e, rows, n, dtype=torch.bfloat16, device=x.device) if valid_rows is not None else \
            torch.empty(e, rows, n, dtype=torch.bfloat16, device=x.device)
        gemm_batched(x, weight, out, rows, n, k, valid_rows=valid_rows, segment_rows=segment_rows)
        ctx.save_for_backward(x, weight, valid_rows)
        ctx.segment_rows = segment_rows
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, weight, valid_rows = ctx.saved_tensors
        e, rows, k = x.shape
        n = weight.shape[1]
        g = grad_out.contiguous()
        grad_x = grad_w = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.zeros_like(x) if valid_rows is not None else torch.empty_like(x)
            gemm_batched(g, weight, grad_x, rows, k, n, b_mn_major=True, valid_rows=valid_rows,
                         segment_rows=ctx.segment_rows)
        if ctx.needs_input_grad[1]:
            # rows past the valid count hold zeros in both operands (padded dispatch buffer), so the full
            # contraction over rows is exact
            main = getattr(weight, "main_grad", None)
            if main is not None:
                gemm_batched(g, x, main, n, k, rows, a_mn_major=True, b_mn_major=True, epilogue=EPI_ACCUM_F32)
                weight.main_grad_written = True
            else:
                grad_w = torch.empty(e, n, k, dtype=torch.bfloat16, device=x.device)
                gemm_batched(g, x, grad_w, n, k, rows, a_mn_major=True, b_mn_major=True)
        return grad_x, grad_w, None, None


def _gemm_batched_swiglu(a, b, gate_up, other, m, n, k, backward: bool, valid_rows, segment_rows) -> None:
    native.call("ajb_gemm_bf16_batched_swiglu", a.data_ptr(), b.data_ptr(), native.ptr(gate_up), other.data_ptr(), a.shape[0],
                m, n, k, a.stride(1), b.stride(1), gate_up.stride(1) if gate_up is not None else 0, other.stride(1),
                a.stride(0), b.stride(0), gate_up.stride(0) if gate_up is not None else 0, other.stride(0),
                int(backward), native.ptr(valid_rows), segment_rows, native.stream_ptr())


class _BatchedSwigluFfnFn(torch.autograd.Function):
    """Stacked SwiGLU experts ``y[e] = (silu(x[e] W1[e]^T) * x[e] W3[e]^T) W2[e]^T`` with the activation and its gradient
    computed by the epilogues of the batched GEMMs around them (``w13`` interleaved per expert)."""

    @staticmethod
    def forward(ctx, x, w13, w2, valid_rows, segment_rows):
        e, rows, k = x.shape
        f2, d_out = w13.shape[1], w2.shape[1]
        x = x.contiguous()
        make = torch.zeros if valid_rows is not None else torch.empty      # skipped row blocks are never written
        gate_up = make(e, rows, f2, dtype=torch.bfloat16, device=x.device)
        act = make(e, rows, f2 // 2, dtype=torch.bfloat16, device=x.device)
        _gemm_batched_swiglu(x, w13, gate_up, act, rows, f2, k, False, valid_rows, segment_rows)
        out = make(e, rows, d_out, dtype=torch.bfloat16, device=x.device)
        gemm_batched(act, w2, out, rows, d_out, f2 // 2, valid_rows=valid_rows, segment_rows=segment_rows)
        ctx.save_for_backward(x, w13, w2, gate_up, act, valid_rows)
        ctx.segment_rows = segment_rows
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x, w13, w2, gate_up, act, valid_rows = ctx.saved_tensors
        e, rows, k = x.shape
        f2, d_out = w13.shape[1], w2.shape[1]
        f = f2 // 2
        g = grad_out.contiguous()
        make = torch.zeros if valid_rows is not None else torch.empty
        d_gate_up = make(e, rows, f2, dtype=torch.bfloat16, device=g.device)
        _gemm_batched_swiglu(g, w2, gate_up, d_gate_up, rows, f, d_out, True, valid_rows, ctx.segment_rows)
        grad_x = grad_w13 = grad_w2 = None
        if ctx.needs_input_grad[0]:
            grad_x = make(e, rows, k, dtype=torch.bfloat16, device=g.device)
            gemm_batched(d_gate_up, w13, grad_x, rows, k, f2, b_mn_major=True, valid_rows=valid_rows,
                         segment_rows=ctx.segment_rows)
        # rows past the valid count hold zeros in both operands of the weight gradients (padded dispatch buffer,
        # zero-initialised intermediates), so the full contraction over rows is exact
        for weight, left, right, n_out, n_in, slot in ((w2, g, act, d_out, f, 2), (w13, d_gate_up, x, f2, k, 1)):
            if not ctx.needs_input_grad[slot]:
                continue
            main = getattr(weight, "main_grad", None)
            if main is not None:
                gemm_batched(left, right, main, n_out, n_in, rows, a_mn_major=True, b_mn_major=True, epilogue=EPI_ACCUM_F32)
                weight.main_grad_written = True
            else:
                grad = torch.empty(e, n_out, n_in, dtype=torch.bfloat16, device=g.device)
                gemm_batched(left, right, grad, n_out, n_in, rows, a_mn_major=True, b_mn_major=True)
                if slot == 2:
                    grad_w2 = grad
                else:
                    grad_w13 = grad
        return grad_x, grad_w13, grad_w2, None, None


def swiglu_ffn_batched(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, valid_rows: torch.Tensor | None = None,
                       segment_rows: int = 0) -> torch.Tensor:
    """Stacked SwiGLU experts ``[E, rows, D] -> [E, rows, D]`` (``w13 [E, 2 F, D]`` interleaved, ``w2 [E, D, F]``)."""
    if (_native(x, "swiglu_ffn_batched") and FUSED_SWIGLU and (w13.shape[1] // 2) % 32 == 0 and x.shape[-1] % 8 == 0
            and w2.shape[1] % 8 == 0 and w13.is_contiguous() and w2.is_contiguous()):
        return _BatchedSwigluFfnFn.apply(x, w13, w2, valid_rows, segment_rows)
    hidden = swiglu_interleaved(linear_batched(x, w13, valid_rows, segment_rows))
    return linear_batched(hidden, w2, valid_rows, segment_rows)


def linear_batched(x: torch.Tensor, weight: torch.Tensor, valid_rows: torch.Tensor | None = None,
                   segment_rows: int = 0) -> torch.Tensor:
    """Stacked-expert projection ``[E, rows, in] x [E, out, in] -> [E, rows, out]``."""
    if _native(x, "linear_batched"):
        return _BatchedLinearFn.apply(x, weight, valid_rows, segment_rows)
    return torch.einsum("erk,enk->ern", x, weight)


class _LinearFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight):
        lead = x.shape[:-1]
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        n, k = weight.shape
        out = torch.empty(x2.shape[0], n, dtype=torch.bfloat16, device=x.device)
        gemm(x2, weight, out, x2.shape[0], n, k)
        ctx.save_for_backward(x2, weight)
        ctx.lead = lead
        return out.view(*lead, n)

    @staticmethod
    def backward(ctx, grad_out):
        x2, weight = ctx.saved_tensors
        n, k = weight.shape
        g2 = grad_out.reshape(-1, n)
        if g2.stride(-1) != 1 or g2.dtype != torch.bfloat16:
            g2 = g2.to(torch.bfloat16).contiguous()
        m = g2.shape[0]
        grad_x = grad_w = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.empty(m, k, dtype=torch.bfloat16, device=g2.device)
            gemm(g2, weight, grad_x, m, k, n, b_mn_major=True)
            grad_x = grad_x.view(*ctx.lead, k)
        if ctx.needs_input_grad[1]:
            main = getattr(weight, "main_grad", None)
            if main is not None:
                # fp32 accumulation straight into the optimizer's gradient buffer
                wgrad_accumulate(g2, x2, main, n, k, m)
                weight.main_grad_written = True
            else:
                grad_w = torch.empty(n, k, dtype=torch.bfloat16, device=g2.device)
                gemm(g2, x2, grad_w, n, k, m, a_mn_major=True, b_mn_major=True)
        return grad_x, grad_w


_SPLITK_WORKSPACE: dict = {}
_SPLITK_RETIRED: list = []      # outgrown workspaces stay allocated: a captured graph may still hold their address
_SKINNY_ROWS = 512


def _splitk_workspace(device: torch.device, floats: int) -> torch.Tensor:
    key = (device.index, )
    workspace = _SPLITK_WORKSPACE.get(key)
    if workspace is None or workspace.numel() < floats:
        if workspace is not None:
            _SPLITK_RETIRED.append(workspace)
        workspace = torch.empty(max(floats, 1 << 22), dtype=torch.float32, device=device)
        _SPLITK_WORKSPACE[key] = workspace
    return workspace
# 129 to 512 rows run on CTA pairs with K slices summed in an L2-resident workspace; AJB_SKINNY_PAIR=0 keeps the
# single-CTA split-K kernel and its separate partial buffers
SKINNY_PAIR_GEMM = os.environ.get("AJB_SKINNY_PAIR", "1") != "0"
_SKINNY_SPLITS: dict = {}


def linear_skinny(x2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """Forward-only ``x2 @ weight.T`` for few rows (decoding): the K range is split over enough CTAs to keep
    every SM streaming weights; fp32 partial products are summed by a second small kernel."""
    m, k = x2.shape
    n = weight.shape[0]
    if m <= 128:
        return _linear_decode(x2, weight)
    if SKINNY_PAIR_GEMM:
        # CTA pairs: every weight byte is fetched once; K slices (chosen by the library) add into an fp32 workspace
        split = _SKINNY_SPLITS.get((m, n, k))
        if split is None:
            split = _SKINNY_SPLITS[(m, n, k)] = int(native.lib().ajb_gemm_skinny_pair_split(m, n, k))
        out = torch.empty(m, n, dtype=torch.bfloat16, device=x2.device)
        workspace = None
        if split > 1:
            workspace = _splitk_workspace(x2.device, m * n)
        native.call("ajb_gemm_bf16_skinny_pair", x2.data_ptr(), weight.data_ptr(), out.data_ptr(), native.ptr(workspace), m, n, k,
                    x2.stride(0), weight.stride(0), split, native.stream_ptr())
        return out
    tiles = ((m + 127) // 128) * ((n + 255) // 256)
    k_blocks = (k + 63) // 64
    want = max(1, min(k_blocks // 4, (148 + tiles - 1) // tiles))
    per = (k_blocks + want - 1) // want
    split = (k_blocks + per - 1) // per
    out = torch.empty(m, n, dtype=torch.bfloat16, device=x2.device)
    workspace = None
    if split > 1:
        workspace = _splitk_workspace(x2.device, split * m * n)
    native.call("ajb_gemm_bf16_splitk", x2.data_ptr(), weight.data_ptr(), out.data_ptr(), native.ptr(workspace), m, n, k,
                x2.stride(0), weight.stride(0), split, native.stream_ptr())
    return out


# Decoding GEMMs with few 128-row weight strips run as one cluster of CTAs per strip that sums its K slices through
# distributed shared memory (csrc/gemm_decode_cluster.cu); AJB_DECODE_CLUSTER=0 keeps them on the split-K kernel pair.
DECODE_CLUSTER_GEMM = os.environ.get("AJB_DECODE_CLUSTER", "1") != "0"
_CLUSTER_SLICES: dict = {}      # (n, k) -> CTAs per weight strip that fit on the device at once, 0 = none


def _linear_decode(x2: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x2 @ weight.T`` for at most 128 rows as ``(weight @ x2.T).T``: weight rows fill the 128-row side of the
    tensor-core tile, ``n / 128`` tiles times a few K slices stream the weights, partial products are tiny."""
    m, k = x2.shape
    n = weight.shape[0]
    tiles = (n + 127) // 128
    k_blocks = (k + 63) // 64
    if DECODE_CLUSTER_GEMM:
        # few 128-row strips: a cluster of CTAs per strip, K slices summed through distributed shared memory
        slices = _CLUSTER_SLICES.get((n, k))
        if slices is None:
            slices = _CLUSTER_SLICES[(n, k)] = int(native.lib().ajb_gemm_decode_cluster_slices(n, k))
        if slices >= 2:
            out = torch.empty(m, n, dtype=torch.bfloat16, device=x2.device)
            native.call("ajb_gemm_bf16_decode_cluster", x2.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k,
                        x2.stride(0), weight.stride(0), out.stride(0), slices, native.stream_ptr())
            return out
    want = max(1, min(k_blocks // 4, (2 * 148 + tiles - 1) // tiles))      # about two CTAs' worth of work per SM
    per = (k_blocks + want - 1) // want
    split = (k_blocks + per - 1) // per
    out = torch.empty(m, n, dtype=torch.bfloat16, device=x2.device)
    workspace = None
    if split > 1:
        workspace = _splitk_workspace(x2.device, split * m * n)
    native.call("ajb_gemm_bf16_decode", x2.data_ptr(), weight.data_ptr(), out.data_ptr(), native.ptr(workspace), m, n, k,
                x2.stride(0), weight.stride(0), split, native.stream_ptr())
    return out


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T`` for a bias-free ``[out, in]`` weight (``ajllm/modeling/layers.py:33``)."""
    if _native(x, "linear"):
        if not torch.is_grad_enabled() and weight.shape[0] % 8 == 0:
            x2 = x.reshape(-1, x.shape[-1])
            if x2.shape[0] <= _SKINNY_ROWS and x2.stride(-1) == 1 and weight.stride(-1) == 1:
                return linear_skinny(x2, weight).view(*x.shape[:-1], weight.shape[0])
        return _LinearFn.apply(x, weight)
    return reference.linear(x, weight)


# ----------------------------------------------------------------------------- RMSNorm (+ residual)

_NORM_BWD_ROWS_PER_BLOCK = 16


def _norm_bwd_partials(rows: int) -> int:
    return max(1, min(1024, (rows + _NORM_BWD_ROWS_PER_BLOCK - 1) // _NORM_BWD_ROWS_PER_BLOCK))


class _AddRmsNormFn(torch.autograd.Function):
    """``h = x + delta`` (``delta`` may be ``None``), ``y = rmsnorm(h) * gain``; returns ``(h, y)``."""

    @staticmethod
    def forward(ctx, x, delta, gain, eps):
        dim = x.shape[-1]
        x2 = x.reshape(-1, dim)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
        if delta is not None:
            h = torch.empty_like(x2)
            d2 = delta.reshape(-1, dim)
        else:
            h, d2 = x2, None
        native.call("ajb_rmsnorm_fwd", x2.data_ptr(), native.ptr(d2), gain.data_ptr(), y.data_ptr(),
                    h.data_ptr() if delta is not None else None, rstd.data_ptr(), rows, dim, float(eps),
                    native.stream_ptr())
        ctx.save_for_backward(h, gain, rstd)
        ctx.has_delta = delta is not None
        ctx.shape = x.shape
        return h.view(x.shape), y.view(x.shape)

    @staticmethod
    def backward(ctx, grad_h, grad_y):
        h, gain, rstd = ctx.saved_tensors
        rows, dim = h.shape
        gy = grad_y.reshape(rows, dim).contiguous()
        gh = None if grad_h is None else grad_h.reshape(rows, dim).contiguous()
        dx = torch.empty_like(h)
        nparts = _norm_bwd_partials(rows)
        partial = torch.empty(nparts, dim, dtype=torch.float32, device=h.device)
        native.call("ajb_rmsnorm_bwd", gy.data_ptr(), h.data_ptr(), gain.data_ptr(), rstd.data_ptr(),
                    native.ptr(gh), dx.data_ptr(), partial.data_ptr(), rows, dim, nparts, native.stream_ptr())
        main = getattr(gain, "main_grad", None)
        grad_gain = None
        if main is not None:
            native.call("ajb_colsum_f32", partial.data_ptr(), main.data_ptr(), nparts, dim, 1, native.stream_ptr())
            gain.main_grad_written = True
        else:
            gsum = torch.zeros(dim, dtype=torch.float32, device=h.device)
            native.call("ajb_colsum_f32", partial.data_ptr(), gsum.data_ptr(), nparts, dim, 0, native.stream_ptr())
            grad_gain = gsum.to(gain.dtype)
        dx = dx.view(ctx.shape)
        return dx, (dx if ctx.has_delta else None), grad_gain, None


def add_rms_norm(x: torch.Tensor, delta: torch.Tensor | None, gain: torch.Tensor, eps: float = 1e-5):
    """Residual add fused with RMSNorm: returns ``(x + delta, rmsnorm(x + delta) * gain)``."""
    if _native(x, "rms_norm"):
        return _AddRmsNormFn.apply(x, delta, gain, eps)
    h = x if delta is None else x + delta
    return h, reference.rms_norm(h, gain, eps)


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    return add_rms_norm(x, None, gain, eps)[1]


# ----------------------------------------------------------------------------- RoPE + attention


def kernel_head_dim(head_dim: int) -> int:
    """Head size the attention kernels run at: they exist for 64- and 128-wide heads, and any other size that is a
    multiple of 8 (the reference's flagship model has 32) is zero-padded up to the next of the two."""
    if head_dim % 8 or head_dim > 128:
        raise ValueError(f"attention head size {head_dim} is not supported on the GPU (a multiple of 8, at most 128)")
    return 64 if head_dim <= 64 else 128


def repack_heads(x: torch.Tensor, heads: int, src_hd: int, dst_hd: int) -> torch.Tensor:
    """``[..., heads * src_hd]`` -> ``[..., heads * dst_hd]``: widen every head with zeros or keep its leading part."""
    lead = x.shape[:-1]
    flat = x.reshape(-1, heads * src_hd)
    if flat.stride(-1) != 1 or flat.stride(0) % 8:
        flat = flat.contiguous()
    out = torch.empty(flat.shape[0], heads * dst_hd, dtype=x.dtype, device=x.device)
    native.call("ajb_repack_heads", flat.data_ptr(), out.data_ptr(), flat.shape[0], heads, src_hd, dst_hd,
                flat.stride(0), out.stride(0), native.stream_ptr())
    return out.view(*lead, heads * dst_hd)


class _RopeAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, num_heads, num_kv_heads, head_dim, causal, use_rope):
        B, T, width = qkv.shape
        assert width == (num_heads + 2 * num_kv_heads) * head_dim
        qkv = qkv.contiguous()
        rows = B * T
        stream = native.stream_ptr()
        if use_rope:
            # rotates the q and k heads of the packed rows in place (positions = row % T)
            native.call("ajb_rope_qk", qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), None, rows, T,
                        num_heads, num_kv_heads, head_dim, width, 0, stream)
        scale = 1.0 / math.sqrt(head_dim)
        khd = kernel_head_dim(head_dim)
        all_heads = num_heads + 2 * num_kv_heads
        if khd != head_dim:
            qkv = repack_heads(qkv, all_heads, head_dim, khd)       # the kernels see zero-padded heads
        out = torch.empty(B, T, num_heads * khd, dtype=torch.bfloat16, device=qkv.device)
        lse = torch.empty(B, num_heads, T, dtype=torch.float32, device=qkv.device)
        native.call("ajb_flash_fwd", qkv.data_ptr(), out.data_ptr(), lse.data_ptr(), B, T, num_heads,
                    num_kv_heads, khd, all_heads * khd, int(causal), scale, stream)
        ctx.save_for_backward(qkv, out, lse, cos, sin)
        ctx.meta = (num_heads, num_kv_heads, head_dim, causal, use_rope, scale)
        return out if khd == head_dim else repack_heads(out, num_heads, khd, head_dim)

    @staticmethod
    def backward(ctx, grad_out):
        qkv, out, lse, cos, sin = ctx.saved_tensors
        num_heads, num_kv_heads, true_head_dim, causal, use_rope, scale = ctx.meta
        head_dim = kernel_head_dim(true_head_dim)
        B, T, width = qkv.shape
        stream = native.stream_ptr()
        grad_out = grad_out.contiguous()
        if head_dim != true_head_dim:
            grad_out = repack_heads(grad_out, num_heads, true_head_dim, head_dim)
        dqkv = torch.empty_like(qkv)
        delta = torch.empty(B, num_heads, T, dtype=torch.float32, device=qkv.device)
        # the fused kernel adds dQ tiles into an fp32 buffer (sum order varies between runs); the
        # bit-reproducible two-kernel path is selected by passing no buffer
        dq_acc = None if DETERMINISTIC_ATTENTION_BACKWARD else \
            torch.empty(B * num_heads * (-(-T // 64) * 64) * head_dim, dtype=torch.float32, device=qkv.device)
        native.call("ajb_flash_bwd", qkv.data_ptr(), out.data_ptr(), grad_out.data_ptr(), lse.data_ptr(),
                    delta.data_ptr(), dqkv.data_ptr(), dq_acc.data_ptr() if dq_acc is not None else None,
                    B, T, num_heads, num_kv_heads, head_dim, width, int(causal), scale, stream)
        if head_dim != true_head_dim:
            dqkv = repack_heads(dqkv, num_heads + 2 * num_kv_heads, head_dim, true_head_dim)
            head_dim, width = true_head_dim, dqkv.shape[-1]
        if use_rope:
            native.call("ajb_rope_qk", dqkv.data_ptr(), cos.data_ptr(), sin.data_ptr(), None, B * T, T,
                        num_heads, num_kv_heads, head_dim, width, 1, stream)
        return dqkv, None, None, None, None, None, None, None


def rope_attention(qkv: torch.Tensor, cos: torch.Tensor | None, sin: torch.Tensor | None, num_heads: int,
                   num_kv_heads: int, head_dim: int, causal: bool = True) -> torch.Tensor:
    """Causal self-attention over a packed ``[B, T, (Hq + 2 Hkv) * hd]`` projection.

    RoPE (interleaved pairs, ``ajllm/modeling/attention.py:50-60``) is applied to the q and k heads when
    tables are given; the result is ``[B, T, Hq * hd]``. On the GPU path the rotation is done in place:
    ``qkv`` must be a buffer the caller no longer needs un-rotated (the output of the projection GEMM).
    """
    B, T, _ = qkv.shape
    if _native(qkv, "rope_attention"):
        use_rope = cos is not None
        if use_rope and (cos.dtype != torch.float32 or sin.dtype != torch.float32 or cos.shape[0] < T):
            raise ValueError("RoPE tables must be fp32 and cover the sequence length")
        dummy = qkv.new_empty(1, dtype=torch.float32)
        return _RopeAttentionFn.apply(qkv, cos if use_rope else dummy, sin if use_rope else dummy,
                                      num_heads, num_kv_heads, head_dim, causal, use_rope)
    q, k, v = split_packed_qkv(qkv, num_heads, num_kv_heads, head_dim)
    if cos is not None:
        pos = torch.arange(T, device=qkv.device)
        q = reference.rope_interleaved(q, cos, sin, pos)
        k = reference.rope_interleaved(k, cos, sin, pos)
    return reference.attention(q, k, v, causal=causal).reshape(B, T, num_heads * head_dim)


def split_packed_qkv(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int):
    lead = qkv.shape[:-1]
    nq, nk = num_heads * head_dim, num_kv_heads * head_dim
    q = qkv[..., :nq].reshape(*lead, num_heads, head_dim)
    k = qkv[..., nq:nq + nk].reshape(*lead, num_kv_heads, head_dim)
    v = qkv[..., nq + nk:].reshape(*lead, num_kv_heads, head_dim)
    return q, k, v


# ----------------------------------------------------------------------------- SwiGLU


class _SwigluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gate_up):
        width = gate_up.shape[-1]
        g2 = gate_up.reshape(-1, width).contiguous()
        act = torch.empty(g2.shape[0], width // 2, dtype=g2.dtype, device=g2.device)
        native.call("ajb_swiglu_fwd", g2.data_ptr(), act.data_ptr(), g2.shape[0], width // 2, native.stream_ptr())
        ctx.save_for_backward(g2)
        ctx.shape = gate_up.shape
        return act.view(*gate_up.shape[:-1], width // 2)

    @staticmethod
    def backward(ctx, grad_act):
        (g2,) = ctx.saved_tensors
        rows, width = g2.shape
        ga = grad_act.reshape(rows, width // 2).contiguous()
        dgu = torch.empty_like(g2)
        native.call("ajb_swiglu_bwd", g2.data_ptr(), ga.data_ptr(), dgu.data_ptr(), rows, width // 2,
                    native.stream_ptr())
        return dgu.view(ctx.shape)


def swiglu_interleaved(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` where even columns are gate and odd columns are up."""
    if _native(gate_up, "swiglu"):
        return _SwigluFn.apply(gate_up)
    return reference.swiglu_interleaved(gate_up)


# SwiGLU computed by the epilogues of the projections around it (csrc/gemm_bf16_pair.cu); AJB_FUSED_SWIGLU=0 keeps the
# three separate steps.
FUSED_SWIGLU = os.environ.get("AJB_FUSED_SWIGLU", "1") != "0"


def _gemm_swiglu(a, b, gate_up, other, m, n, k, backward: bool) -> None:
    native.call("ajb_gemm_bf16_swiglu", a.data_ptr(), b.data_ptr(), native.ptr(gate_up), other.data_ptr(), m, n, k,
                a.stride(0), b.stride(0), gate_up.stride(0) if gate_up is not None else 0, other.stride(0),
                int(backward), native.stream_ptr())


class _SwigluFfnFn(torch.autograd.Function):
    """``(silu(x W1^T) * x W3^T) W2^T`` with W1 / W3 rows interleaved in ``w13``: the activation leaves the first
    projection's epilogue, and in the backward pass the gradient of ``gate_up`` leaves the epilogue of
    ``d_out @ W2`` without ``d_act`` ever being stored."""

    @staticmethod
    def run_forward(x, w13, w2, keep: bool):
        """Returns ``(out, x2, gate_up, act)``; without ``keep`` the pre-activation is never written."""
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        m, k = x2.shape
        f2 = w13.shape[0]
        d_out = w2.shape[0]
        gate_up = torch.empty(m, f2, dtype=torch.bfloat16, device=x.device) if keep else None
        act = torch.empty(m, f2 // 2, dtype=torch.bfloat16, device=x.device)
        _gemm_swiglu(x2, w13, gate_up, act, m, f2, k, backward=False)
        out = torch.empty(m, d_out, dtype=torch.bfloat16, device=x.device)
        gemm(act, w2, out, m, d_out, f2 // 2)
        return out.view(*x.shape[:-1], d_out), x2, gate_up, act

    @staticmethod
    def forward(ctx, x, w13, w2):
        out, x2, gate_up, act = _SwigluFfnFn.run_forward(x, w13, w2, keep=True)
        ctx.save_for_backward(x2, w13, w2, gate_up, act)
        ctx.lead = x.shape[:-1]
        return out

    @staticmethod
    def backward(ctx, grad_out):
        x2, w13, w2, gate_up, act = ctx.saved_tensors
        m, k = x2.shape
        f2 = w13.shape[0]
        f = f2 // 2
        d_out = w2.shape[0]
        g2 = grad_out.reshape(-1, d_out)
        if g2.stride(-1) != 1 or g2.dtype != torch.bfloat16:
            g2 = g2.to(torch.bfloat16).contiguous()
        d_gate_up = torch.empty(m, f2, dtype=torch.bfloat16, device=g2.device)
        _gemm_swiglu(g2, w2, gate_up, d_gate_up, m, f, d_out, backward=True)
        grad_x = grad_w13 = grad_w2 = None
        if ctx.needs_input_grad[2]:
            main = getattr(w2, "main_grad", None)
            if main is not None:
                wgrad_accumulate(g2, act, main, d_out, f, m)
                w2.main_grad_written = True
            else:
                grad_w2 = torch.empty(d_out, f, dtype=torch.bfloat16, device=g2.device)
                gemm(g2, act, grad_w2, d_out, f, m, a_mn_major=True, b_mn_major=True)
        if ctx.needs_input_grad[0]:
            grad_x = torch.empty(m, k, dtype=torch.bfloat16, device=g2.device)
            gemm(d_gate_up, w13, grad_x, m, k, f2, b_mn_major=True)
            grad_x = grad_x.view(*ctx.lead, k)
        if ctx.needs_input_grad[1]:
            main = getattr(w13, "main_grad", None)
            if main is not None:
                wgrad_accumulate(d_gate_up, x2, main, f2, k, m)
                w13.main_grad_written = True
            else:
                grad_w13 = torch.empty(f2, k, dtype=torch.bfloat16, device=g2.device)
                gemm(d_gate_up, x2, grad_w13, f2, k, m, a_mn_major=True, b_mn_major=True)
        return grad_x, grad_w13, grad_w2


def swiglu_ffn(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor) -> torch.Tensor:
    """The SwiGLU feed-forward block ``W2(silu(W1 x) * W3 x)`` (``ajllm/modeling/activations.py:15-27``) for an
    interleaved ``w13``. On the GPU the activation and its gradient are computed inside the GEMM epilogues when the
    shapes allow (more than 128 rows, hidden width a multiple of 32); otherwise as three steps."""
    if _native(x, "swiglu_ffn"):
        rows = x.numel() // x.shape[-1]
        f = w13.shape[0] // 2
        fused = (FUSED_SWIGLU and rows > _SKINNY_ROWS and f % 32 == 0 and x.shape[-1] % 8 == 0 and w2.shape[0] % 8 == 0
                 and w13.stride(-1) == 1 and w2.stride(-1) == 1 and w2.stride(0) % 8 == 0 and w13.stride(0) % 8 == 0)
        if fused:
            if torch.is_grad_enabled() and (x.requires_grad or w13.requires_grad or w2.requires_grad):
                return _SwigluFfnFn.apply(x, w13, w2)
            return _SwigluFfnFn.run_forward(x, w13, w2, keep=False)[0]
    return linear(swiglu_interleaved(linear(x, w13)), w2)


def linear_swiglu(x: torch.Tensor, w13: torch.Tensor) -> torch.Tensor:
    """``silu(x W1^T) * x W3^T`` for an interleaved ``w13``. Without autograd, on more than a few hundred rows, the
    activation leaves the projection's epilogue and the pre-activation is never written."""
    if (_native(x, "linear_swiglu") and FUSED_SWIGLU and not (torch.is_grad_enabled() and (x.requires_grad or w13.requires_grad))
            and x.numel() // x.shape[-1] > _SKINNY_ROWS and (w13.shape[0] // 2) % 32 == 0 and x.shape[-1] % 8 == 0
            and w13.stride(-1) == 1 and w13.stride(0) % 8 == 0):
        x2 = x.reshape(-1, x.shape[-1])
        if x2.stride(-1) != 1:
            x2 = x2.contiguous()
        act = torch.empty(x2.shape[0], w13.shape[0] // 2, dtype=torch.bfloat16, device=x.device)
        _gemm_swiglu(x2, w13, None, act, x2.shape[0], w13.shape[0], x2.shape[1], backward=False)
        return act.view(*x.shape[:-1], act.shape[-1])
    return swiglu_interleaved(linear(x, w13))


class _SiluFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        flat = x.contiguous()
        out = torch.empty_like(flat)
        native.call("ajb_silu", flat.data_ptr(), None, out.data_ptr(), flat.numel(), native.stream_ptr())
        ctx.save_for_backward(flat)
        return out

    @staticmethod
    def backward(ctx, grad_out):
        (flat,) = ctx.saved_tensors
        g = grad_out.contiguous()
        dx = torch.empty_like(flat)
        native.call("ajb_silu", flat.data_ptr(), g.data_ptr(), dx.data_ptr(), flat.numel(), native.stream_ptr())
        return dx


def silu(x: torch.Tensor) -> torch.Tensor:
    """``x * sigmoid(x)`` (``ajllm/modeling/activations.py:11``)."""
    if _native(x, "silu") and x.numel() % 8 == 0:
        return _SiluFn.apply(x)
    return reference.silu(x)


# ----------------------------------------------------------------------------- embedding


class _EmbeddingFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, table):
        flat = ids.reshape(-1).to(torch.int64).contiguous()
        vocab, dim = table.shape
        out = torch.empty(flat.numel(), dim, dtype=table.dtype, device=table.device)
        native.call("ajb_embedding_fwd", flat.data_ptr(), table.data_ptr(), out.data_ptr(), flat.numel(), dim,
                    vocab, native.stream_ptr())
        ctx.save_for_backward(flat, table)
        return out.view(*ids.shape, dim)

    @staticmethod
    def backward(ctx, grad_out):
        flat, table = ctx.saved_tensors
        vocab, dim = table.shape
        g = grad_out.reshape(-1, dim).contiguous()
        main = getattr(table, "main_grad", None)
        if main is not None:
            native.call("ajb_embedding_bwd", flat.data_ptr(), g.data_ptr(), main.data_ptr(), flat.numel(), dim,
                        vocab, native.stream_ptr())
            table.main_grad_written = True
            return None, None
        acc = torch.zeros(vocab, dim, dtype=torch.float32, device=g.device)
        native.call("ajb_embedding_bwd", flat.data_ptr(), g.data_ptr(), acc.data_ptr(), flat.numel(), dim, vocab,
                    native.stream_ptr())
        return None, acc.to(table.dtype)


def embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """Row gather ``table[ids]`` (``ajllm/modeling/layers.py:53``)."""
    if _native(table, "embedding"):
        return _EmbeddingFn.apply(ids, table)
    return table[ids]


# ----------------------------------------------------------------------------- LM head + cross-entropy

_CE_ROWS_PER_CHUNK = 8192


def _logits_chunk(rows: int, vocab: int, device) -> torch.Tensor:
    """``[rows, vocab]`` bf16 scratch whose row pitch is a multiple of 8 elements: the logits are read back by TMA as a
    GEMM operand, which needs 16-byte aligned rows whatever the vocabulary size. The columns past ``vocab`` are never
    read (the tensor maps end at ``vocab``)."""
    pitch = (vocab + 7) // 8 * 8
    return torch.empty(rows, pitch, dtype=torch.bfloat16, device=device)[:, :vocab]


class _LinearCrossEntropyFn(torch.autograd.Function):
    """Mean cross-entropy of ``hidden @ weight.T`` without keeping the ``[tokens, vocab]`` logits.

    Row chunks go through GEMM -> in-place softmax-minus-onehot -> the two gradient GEMMs while still in
    the forward pass, so the only saved tensors are ``d hidden`` and (optionally) ``d weight``.
    """

    @staticmethod
    def forward(ctx, hidden, weight, targets, loss_scale):
        dim = hidden.shape[-1]
        h2 = hidden.reshape(-1, dim).contiguous()
        tgt = targets.reshape(-1).to(torch.int64).contiguous()
        rows, vocab = h2.shape[0], weight.shape[0]
        stream = native.stream_ptr()
        loss_sum = torch.zeros(1, dtype=torch.float32, device=h2.device)
        grad_h = torch.empty_like(h2)
        main = getattr(weight, "main_grad", None)
        grad_w = main if main is not None else torch.zeros(vocab, dim, dtype=torch.float32, device=h2.device)
        inv = float(loss_scale) / rows
        chunk = min(rows, _CE_ROWS_PER_CHUNK)
        logits = _logits_chunk(chunk, vocab, h2.device)
        for start in range(0, rows, chunk):
            r = min(chunk, rows - start)
            hs = h2[start:start + r]
            gemm(hs, weight, logits, r, vocab, dim)
            native.call("ajb_ce_fwd_bwd", logits.data_ptr(), tgt[start:start + r].data_ptr(), loss_sum.data_ptr(),
                        r, vocab, logits.stride(0), inv, 1, stream)
            gemm(logits, weight, grad_h[start:start + r], r, dim, vocab, b_mn_major=True)
            gemm(logits, hs, grad_w, vocab, dim, r, a_mn_major=True, b_mn_major=True, epilogue=EPI_ACCUM_F32)
        ctx.save_for_backward(grad_h, None if main is not None else grad_w)
        ctx.uses_main = main is not None
        if main is not None:
            weight.main_grad_written = True
        ctx.hshape = hidden.shape
        ctx.wdtype = weight.dtype
        return (loss_sum / rows).reshape(())

    @staticmethod
    def backward(ctx, grad_loss):
        grad_h, grad_w = ctx.saved_tensors
        # the chunk gradients were scaled by loss_scale/rows already; grad_loss multiplies on top
        gh = grad_h.view(ctx.hshape) * grad_loss.to(grad_h.dtype)
        gw = None if ctx.uses_main else (grad_w * grad_loss).to(ctx.wdtype)
        return gh, gw, None, None


def _linear_cross_entropy_eval(hidden, weight, targets) -> torch.Tensor:
    dim = hidden.shape[-1]
    h2 = hidden.reshape(-1, dim).contiguous()
    tgt = targets.reshape(-1).to(torch.int64).contiguous()
    rows, vocab = h2.shape[0], weight.shape[0]
    loss_sum = torch.zeros(1, dtype=torch.float32, device=h2.device)
    chunk = min(rows, _CE_ROWS_PER_CHUNK)
    logits = _logits_chunk(chunk, vocab, h2.device)
    for start in range(0, rows, chunk):
        r = min(chunk, rows - start)
        gemm(h2[start:start + r], weight, logits, r, vocab, dim)
        native.call("ajb_ce_fwd_bwd", logits.data_ptr(), tgt[start:start + r].data_ptr(), loss_sum.data_ptr(),
                    r, vocab, logits.stride(0), 0.0, 0, native.stream_ptr())
    return (loss_sum / rows).reshape(())


def linear_cross_entropy(hidden: torch.Tensor, weight: torch.Tensor, targets: torch.Tensor,
                         loss_scale: float = 1.0) -> torch.Tensor:
    """Mean CE of the LM head (``ajllm/modeling/transformer.py:123-126`` followed by
    ``ajllm/training/losses.py:8-18``). ``loss_scale`` pre-multiplies the gradients only (used for
    gradient accumulation); the returned loss is unscaled.

    On the GPU the gradients are produced during the forward call, so the caller must backpropagate the
    returned loss with a unit (or scalar) upstream gradient.
    """
    if _native(hidden, "linear_cross_entropy"):
        if torch.is_grad_enabled() and (hidden.requires_grad or weight.requires_grad):
            return _LinearCrossEntropyFn.apply(hidden, weight, targets, loss_scale)
        return _linear_cross_entropy_eval(hidden, weight, targets)
    logits = reference.linear(hidden, weight)
    loss = reference.cross_entropy(logits, targets)
    if loss_scale != 1.0:
        # same value, scaled gradient
        loss = loss.detach() + (loss - loss.detach()) * loss_scale
    return loss


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean CE over materialised logits (evaluation path)."""
    if _is_cuda(logits) and logits.dtype == torch.bfloat16 and not logits.requires_grad:
        flat = logits.reshape(-1, logits.shape[-1]).contiguous()
        tgt = targets.reshape(-1).to(torch.int64).contiguous()
        loss_sum = torch.zeros(1, dtype=torch.float32, device=flat.device)
        native.call("ajb_ce_fwd_bwd", flat.data_ptr(), tgt.data_ptr(), loss_sum.data_ptr(), flat.shape[0],
                    flat.shape[1], flat.stride(0), 0.0, 0, native.stream_ptr())
        return (loss_sum / flat.shape[0]).reshape(())
    return reference.cross_entropy(logits, targets)


# ----------------------------------------------------------------------------- paged attention (serving)


def paged_attention_ragged(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor,
                           block_tables: torch.Tensor, context_lens: torch.Tensor, q_lens: torch.Tensor,
                           q_lens_host: list[int], context_lens_host: list[int]) -> torch.Tensor:
    """Attention of ragged new tokens over a paged KV cache.

    ``q`` is ``[total_new_tokens, Hq, hd]``, concatenated per sequence; sequence ``i`` contributes
    ``q_lens[i]`` rows which sit at positions ``context_lens[i] - q_lens[i] ..`` of that sequence and
    attend causally to its first ``context_lens[i]`` cached tokens. Caches are
    ``[num_blocks, block, Hkv, hd]``. Returns ``[total_new_tokens, Hq, hd]``.
    """
    if _is_cuda(q) and q.dtype == torch.bfloat16 and native.available() and hasattr(native.lib(), "ajb_paged_attention"):
        from ajllm_b200.ops import serving
        return serving.paged_attention(q, key_cache, value_cache, block_tables, context_lens, q_lens,
                                       q_lens_host, context_lens_host)
    out = torch.empty_like(q)
    block = key_cache.shape[1]
    cursor = 0
    for i, (n, length) in enumerate(zip(q_lens_host, context_lens_host)):
        nblk = (length + block - 1) // block
        ids = block_tables[i, :nblk].long()
        keys = key_cache[ids].reshape(nblk * block, *key_cache.shape[2:])[:length]
        values = value_cache[ids].reshape(nblk * block, *value_cache.shape[2:])[:length]
        out[cursor:cursor + n] = reference.attention(q[cursor:cursor + n][None], keys[None], values[None],
                                                     causal=True)[0]
        cursor += n
    return out
