"""Plain PyTorch statements of every op, used as the CPU path and as the numerics oracle.

Each function states the math of the matching reference op in fp32 and is what the sm_100a kernels
are tested against. Citations give the reference's definition of the same op.
"""

from __future__ import annotations

import math

import torch


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``x @ weight.T`` with ``weight`` stored ``[out, in]`` (``ajllm/modeling/layers.py:33``)."""
    return x @ weight.transpose(-1, -2)


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """fp32 RMS normalisation, cast back to the input dtype (``ajllm/modeling/layers.py:70-74``)."""
    xf = x.float()
    inv = torch.rsqrt(xf.square().mean(dim=-1, keepdim=True) + eps)
    return (xf * inv * gain.float()).to(x.dtype)


def rope_tables(head_dim: int, positions: int, theta: float, device=None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[positions, head_dim/2]``; angle = pos * theta^(-2i/head_dim)
    (``ajllm/modeling/attention.py:43-46``)."""
    if head_dim % 2:
        raise ValueError("RoPE requires an even attention head dimension")
    idx = torch.arange(0, head_dim, 2, device=device, dtype=torch.float32)
    freq = theta ** (-idx / head_dim)
    ang = torch.arange(positions, device=device, dtype=torch.float32)[:, None] * freq[None, :]
    return torch.cos(ang), torch.sin(ang)


def rope_interleaved(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Rotate pairs ``(x[2i], x[2i+1])`` (``ajllm/modeling/attention.py:50-60``).

    ``x`` is ``[..., T, heads, head_dim]`` with ``positions`` broadcastable to ``[..., T]``.
    """
    c = cos[positions].unsqueeze(-2).to(torch.float32)
    s = sin[positions].unsqueeze(-2).to(torch.float32)
    xf = x.float()
    even, odd = xf[..., 0::2], xf[..., 1::2]
    out = torch.stack((even * c - odd * s, even * s + odd * c), dim=-1).flatten(-2)
    return out.to(x.dtype)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              scale: float | None = None) -> torch.Tensor:
    """Softmax attention with grouped KV heads.

    ``q`` is ``[B, T, Hq, hd]``, ``k``/``v`` are ``[B, S, Hkv, hd]`` with ``Hq % Hkv == 0``; query head
    ``h`` reads KV head ``h // (Hq // Hkv)``. With ``causal`` the query at ``t`` sees keys
    ``<= t + (S - T)``. Matches ``scaled_dot_product_attention`` in ``ajllm/modeling/attention.py:20-33``
    for ``Hq == Hkv``.
    """
    B, T, Hq, hd = q.shape
    S, Hkv = k.shape[1], k.shape[2]
    group = Hq // Hkv
    scale = scale if scale is not None else 1.0 / math.sqrt(hd)
    qf = q.float().permute(0, 2, 1, 3)                       # B Hq T hd
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    vf = v.float().permute(0, 2, 1, 3).repeat_interleave(group, dim=1)
    scores = (qf @ kf.transpose(-1, -2)) * scale
    if causal:
        rows = torch.arange(T, device=q.device)[:, None] + (S - T)
        cols = torch.arange(S, device=q.device)[None, :]
        scores = scores.masked_fill(cols > rows, float("-inf"))
    probs = torch.softmax(scores, dim=-1)
    out = probs @ vf
    return out.permute(0, 2, 1, 3).to(q.dtype)


def attention_lse(q: torch.Tensor, k: torch.Tensor, causal: bool = True) -> torch.Tensor:
    """Row log-sum-exp of the scaled scores, ``[B, Hq, T]`` (what the flash forward also returns)."""
    B, T, Hq, hd = q.shape
    S, Hkv = k.shape[1], k.shape[2]
    kf = k.float().permute(0, 2, 1, 3).repeat_interleave(Hq // Hkv, dim=1)
    scores = (q.float().permute(0, 2, 1, 3) @ kf.transpose(-1, -2)) / math.sqrt(hd)
    if causal:
        rows = torch.arange(T, device=q.device)[:, None] + (S - T)
        scores = scores.masked_fill(torch.arange(S, device=q.device)[None, :] > rows, float("-inf"))
    return torch.logsumexp(scores, dim=-1)


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` (``ajllm/modeling/activations.py:25``), computed in fp32."""
    return (silu(gate.float()) * up.float()).to(gate.dtype)


def swiglu_interleaved(gate_up: torch.Tensor) -> torch.Tensor:
    """Same, for a tensor whose last dim interleaves gate (even) and up (odd) columns."""
    return swiglu(gate_up[..., 0::2], gate_up[..., 1::2])


def cross_entropy(logits: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    """Mean token cross-entropy with fp32 accumulation (``ajllm/training/losses.py:8-18``; the
    reference runs in the logits dtype, here the reduction is always fp32)."""
    flat = logits.reshape(-1, logits.shape[-1]).float()
    tgt = targets.reshape(-1)
    lse = torch.logsumexp(flat, dim=-1)
    picked = flat.gather(1, tgt[:, None]).squeeze(1)
    return (lse - picked).mean()


def adamw_update(param: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int,
                 lr: float, beta1: float, beta2: float, eps: float, weight_decay: float,
                 grad_scale: float = 1.0) -> None:
    """In-place AdamW in the reference's order: Adam step first, then ``p *= 1 - lr*wd`` applied to
    the already-updated parameter (``ajllm/training/optimizers.py:46-54``)."""
    g = grad.float() * grad_scale
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    step_size = lr * math.sqrt(1 - beta2**step) / (1 - beta1**step)
    param.addcdiv_(m, v.sqrt().add_(eps), value=-step_size)
    param.mul_(1 - lr * weight_decay)


def top_p_filter(probs: torch.Tensor, top_p: float) -> torch.Tensor:
    """Zero every token whose *preceding* sorted cumulative mass is already ``>= top_p`` and
    renormalise (``ajllm/generation/sampling.py:15-21``)."""
    if not 0 < top_p <= 1:
        raise ValueError("top_p must be in (0, 1]")
    ordered, index = torch.sort(probs, descending=True, dim=-1)
    before = torch.cumsum(ordered, dim=-1) - ordered
    ordered = ordered.masked_fill(before >= top_p, 0.0)
    ordered = ordered / ordered.sum(dim=-1, keepdim=True)
    return torch.zeros_like(probs).scatter(-1, index, ordered)


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_tables: torch.Tensor,
                    context_lens: torch.Tensor, scale: float | None = None) -> torch.Tensor:
    """Decode/verify attention over a paged KV cache.

    ``q`` is ``[num_seqs, q_len, Hq, hd]`` (``q_len`` > 1 for speculative verification: query row ``j``
    sits at position ``context_len - q_len + j``); caches are ``[num_blocks, block, Hkv, hd]``;
    ``block_tables`` is ``[num_seqs, max_blocks]``; ``context_lens`` counts the cached tokens
    including the ``q_len`` newest ones.
    """
    n, qlen, Hq, hd = q.shape
    block = k_cache.shape[1]
    out = torch.empty_like(q)
    for i in range(n):
        L = int(context_lens[i])
        nblk = (L + block - 1) // block
        ids = block_tables[i, :nblk].long()
        ks = k_cache[ids].reshape(nblk * block, *k_cache.shape[2:])[:L]
        vs = v_cache[ids].reshape(nblk * block, *v_cache.shape[2:])[:L]
        out[i] = attention(q[i:i + 1], ks[None], vs[None], causal=True, scale=scale)[0]
    return out


def quantize_weight_fp8_blocks(weight: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """e4m3 weights with one fp32 scale per ``block x block`` tile: ``w ≈ q * scale``."""
    out_f, in_f = weight.shape
    rows, cols = (out_f + block - 1) // block, (in_f + block - 1) // block
    padded = torch.zeros(rows * block, cols * block, dtype=torch.float32, device=weight.device)
    padded[:out_f, :in_f] = weight.float()
    tiles = padded.view(rows, block, cols, block)
    amax = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-12)
    scale = amax / 448.0
    q = (tiles / scale[:, None, :, None]).clamp(-448.0, 448.0).view(rows * block, cols * block)
    return q[:out_f, :in_f].to(torch.float8_e4m3fn), scale


def quantize_activation_fp8_rows(x: torch.Tensor, group: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """Per-token e4m3 activations with one fp32 scale per ``1 x group`` slice of the feature dim."""
    rows, feat = x.shape
    groups = (feat + group - 1) // group
    padded = torch.zeros(rows, groups * group, dtype=torch.float32, device=x.device)
    padded[:, :feat] = x.float()
    g = padded.view(rows, groups, group)
    scale = g.abs().amax(dim=-1).clamp_min(1e-12) / 448.0
    q = (g / scale[..., None]).clamp(-448.0, 448.0).view(rows, groups * group)[:, :feat]
    return q.to(torch.float8_e4m3fn), scale


def fp8_block_linear(xq: torch.Tensor, x_scale: torch.Tensor, wq: torch.Tensor, w_scale: torch.Tensor,
                     block: int = 128) -> torch.Tensor:
    """Dequantise-then-matmul oracle for the block-scaled fp8 GEMM; returns fp32 ``[rows, out]``."""
    rows, feat = xq.shape
    out_f = wq.shape[0]
    xs = x_scale.repeat_interleave(block, dim=1)[:, :feat]
    ws = w_scale.repeat_interleave(block, dim=0).repeat_interleave(block, dim=1)[:out_f, :feat]
    return (xq.float() * xs) @ (wq.float() * ws).t()
