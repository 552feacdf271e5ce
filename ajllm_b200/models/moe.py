"""Mixture-of-experts feed-forward with expert parallelism.

The reference has no MoE; this module defines the semantics that the kernels and the multi-rank
paths are tested against:

* router: ``probs = softmax(x @ Wr.T)`` in fp32, top-``k`` experts per token, gate = the selected
  probabilities (renormalised to sum to one when ``normalize_gates``);
* auxiliary load-balance loss ``coef * E * sum_e f_e * P_e`` with ``f_e`` the fraction of the ``N*k``
  assignments that chose expert ``e`` and ``P_e`` the mean router probability of ``e``;
* capacity: every expert accepts at most ``C = ceil(capacity_factor * N * k / E)`` assignments from the
  ``N`` tokens routed by one rank, taken in (token, choice) order; the rest are dropped (their gate
  contributes nothing, no renormalisation);
* experts: SwiGLU with interleaved ``[E, 2F, D]`` input weights and ``[E, D, F]`` output weights;
* shared experts: ``S`` always-on SwiGLU experts, stored as one SwiGLU of width ``S*F`` (the sum of
  ``S`` width-``F`` SwiGLUs equals one width-``S*F`` SwiGLU);
* output ``sum_k gate_k * expert_{e_k}(x) + shared(x)``.

With expert parallelism the experts are split evenly over the EP group and the fixed-capacity
``[E, C, D]`` dispatch buffer crosses ranks with one all-to-all each way.
"""

from __future__ import annotations

import math

import torch
import torch.distributed as dist
from torch import nn

from ajllm_b200 import ops
from ajllm_b200.models.feed_forward import SwiGLU, deinterleave_rows, interleave_rows
from ajllm_b200.models.layers import InitSpec, init_matrix_
from ajllm_b200.ops import native


def route_tokens(logits: torch.Tensor, top_k: int, capacity: int, normalize_gates: bool = True,
                 stride: int | None = None):
    """Routing decision for ``[N, E]`` router logits.

    Returns ``(gates [N,k] fp32, experts [N,k], slots [N,k], aux_terms)`` where ``slots`` is the row of
    the ``[E * stride]`` dispatch buffer an assignment lands in (``stride`` defaults to ``capacity``; a
    larger stride pads every expert's region), or ``-1`` when it was dropped, and
    ``aux_terms = (f [E], P [E], kept [E])`` with ``kept`` the int32 number of assignments every expert accepted
    (``min(count, capacity)``). On a GPU the slot assignment is one kernel (one CTA per expert scans
    the assignments in order); gates and probabilities stay in autograd.
    """
    tokens, num_experts = logits.shape
    stride = capacity if stride is None else stride
    probs = torch.softmax(logits.float(), dim=-1)
    gates, experts = torch.topk(probs, top_k, dim=-1)
    if normalize_gates:
        gates = gates / gates.sum(dim=-1, keepdim=True)
    flat_expert = experts.reshape(-1)
    if logits.is_cuda and native.available():
        flat32 = flat_expert.to(torch.int32).contiguous()
        slots = torch.empty_like(flat32)
        kept = torch.empty(num_experts, dtype=torch.int32, device=logits.device)
        native.call("ajb_moe_assign_slots", flat32.data_ptr(), flat32.numel(), num_experts, capacity, stride,
                    slots.data_ptr(), kept.data_ptr(), native.stream_ptr())
        counts = torch.bincount(flat_expert, minlength=num_experts)
        slots = slots.long()
    else:
        kept = None
        order = torch.argsort(flat_expert, stable=True)
        counts = torch.bincount(flat_expert, minlength=num_experts)
        starts = torch.cumsum(counts, 0) - counts
        position = torch.empty_like(flat_expert)
        position[order] = torch.arange(flat_expert.numel(), device=logits.device) - starts[flat_expert[order]]
        slots = torch.where(position < capacity, flat_expert * stride + position, torch.full_like(position, -1))
    fraction = counts.float() / float(tokens * top_k)
    mean_prob = probs.mean(dim=0)
    if kept is None:
        kept = counts.clamp(max=capacity).to(torch.int32)
    return gates, experts, slots.reshape(tokens, top_k), (fraction, mean_prob, kept)


def capacity_for(tokens: int, top_k: int, num_experts: int, capacity_factor: float) -> int:
    return max(1, math.ceil(capacity_factor * tokens * top_k / num_experts))


class _AllToAll(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        out = torch.empty_like(x)
        dist.all_to_all_single(out, x.contiguous(), group=group)
        return out

    @staticmethod
    def backward(ctx, grad):
        out = torch.empty_like(grad)
        dist.all_to_all_single(out, grad.contiguous(), group=ctx.group)
        return out, None


class ExpertBank(nn.Module):
    """``num_local`` SwiGLU experts applied to ``[num_local, rows, D]``."""

    def __init__(self, num_total: int, d_model: int, d_ff: int, init: InitSpec, first: int = 0,
                 num_local: int | None = None) -> None:
        super().__init__()
        num_local = num_total if num_local is None else num_local
        w13 = torch.empty(num_local, 2 * d_ff, d_model)
        w2 = torch.empty(num_local, d_model, d_ff)
        # every rank draws all experts so that the global weights do not depend on the EP layout
        for e in range(num_total):
            g, u, d = torch.empty(d_ff, d_model), torch.empty(d_ff, d_model), torch.empty(d_model, d_ff)
            init_matrix_(g, d_model, d_ff, init)
            init_matrix_(d, d_ff, d_model, init)
            init_matrix_(u, d_model, d_ff, init)
            if first <= e < first + num_local:
                w13[e - first], w2[e - first] = interleave_rows(g, u), d
        self.w13 = nn.Parameter(w13)
        self.w2 = nn.Parameter(w2)

    def forward(self, x: torch.Tensor, valid_rows: torch.Tensor | None = None, segment_rows: int = 0) -> torch.Tensor:
        """All local experts in one batched GEMM per projection; with ``valid_rows`` (rows in use per
        capacity segment) the kernels skip row blocks that hold only padding."""
        return ops.swiglu_ffn_batched(x, self.w13, self.w2, valid_rows, segment_rows)


class MoEFeedForward(nn.Module):
    def __init__(self, d_model: int, moe: dict, init: InitSpec = InitSpec(), ep=None) -> None:
        super().__init__()
        self.num_experts = int(moe["num_experts"])
        self.top_k = int(moe["top_k"])
        self.d_ff = int(moe["d_ff"])
        self.shared_experts = int(moe.get("shared_experts", 0))
        self.aux_loss_coef = float(moe.get("aux_loss_coef", 0.0))
        self.capacity_factor = float(moe.get("capacity_factor", 1.25))
        self.normalize_gates = bool(moe.get("normalize_gates", True))
        self.ep = ep
        ep_size = ep.size if ep is not None else 1
        if self.num_experts % ep_size:
            raise ValueError("expert parallel size must divide num_experts")
        self.num_local = self.num_experts // ep_size
        self.router = nn.Parameter(torch.empty(self.num_experts, d_model))
        init_matrix_(self.router.data, d_model, self.num_experts, init)
        first = (ep.rank if ep is not None else 0) * self.num_local
        self.experts = ExpertBank(self.num_experts, d_model, self.d_ff, init, first, self.num_local)
        self.shared = SwiGLU(d_model, self.shared_experts * self.d_ff, init) if self.shared_experts else None
        self.last_aux_loss: torch.Tensor | None = None
        self.last_dropped_fraction: float | None = None
        self._register_state_dict_hook(self._on_save)
        self._register_load_state_dict_pre_hook(self._on_load)

    # checkpoint keys: router.weight, experts.{w1,w2,w3}.weight as [E, ...] stacks, shared.{w1,w2,w3}.weight
    def _all_experts(self, local: torch.Tensor) -> torch.Tensor:
        if self.ep is None or self.ep.size == 1:
            return local
        return self.ep.all_gather_cat(local.contiguous(), 0)

    def _on_save(self, module, state, prefix, local_metadata):
        state[prefix + "router.weight"] = state.pop(prefix + "router")
        w13 = self._all_experts(state.pop(prefix + "experts.w13"))
        w2 = self._all_experts(state.pop(prefix + "experts.w2"))
        gate_up = w13.reshape(w13.shape[0], w13.shape[1] // 2, 2, w13.shape[2])
        state[prefix + "experts.w1.weight"] = gate_up[:, :, 0].clone()
        state[prefix + "experts.w3.weight"] = gate_up[:, :, 1].clone()
        state[prefix + "experts.w2.weight"] = w2.clone()
        return state

    def _on_load(self, state, prefix, *unused):
        if prefix + "router.weight" in state:
            state[prefix + "router"] = state.pop(prefix + "router.weight")
        k1, k2, k3 = (prefix + f"experts.w{i}.weight" for i in (1, 2, 3))
        first = (self.ep.rank if self.ep is not None else 0) * self.num_local
        mine = slice(first, first + self.num_local)
        if k1 in state and k3 in state:
            gate, up = state.pop(k1)[mine], state.pop(k3)[mine]
            state[prefix + "experts.w13"] = torch.stack((gate, up), dim=2).reshape(
                gate.shape[0], 2 * gate.shape[1], gate.shape[2]).contiguous()
        if k2 in state:
            state[prefix + "experts.w2"] = state.pop(k2)[mine].contiguous()

    def _forward_fused(self, flat, gates, slots, counts, stride, exchange) -> torch.Tensor:
        """Expert-parallel path over symmetric memory: rows go straight to the owning rank's expert-major buffer,
        experts run as batched GEMMs that skip padding, outputs are read back and gate-weighted in one kernel.
        ``counts`` (int32 ``[E]``) are the rows every expert accepted from this rank; nothing here waits for the host."""
        from ajllm_b200.parallel import moe_exchange

        slots32 = slots.to(torch.int32).contiguous()
        grouped = moe_exchange.dispatch(flat, slots32, counts, exchange, self.num_local, stride)
        valid = exchange.received_counts(self.num_local)
        result = self.experts(grouped, valid, stride)
        combined = moe_exchange.combine(result, gates.float().contiguous(), slots32, exchange, self.num_local, stride)
        if self.shared is not None:
            combined = combined + self.shared(flat)
        return combined

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        shape = x.shape
        flat = x.reshape(-1, shape[-1])
        tokens, dim = flat.shape
        capacity = capacity_for(tokens, self.top_k, self.num_experts, self.capacity_factor)
        on_gpu = flat.is_cuda and flat.dtype == torch.bfloat16
        # on a GPU every expert's region is padded to whole 128-row tiles so the batched GEMM can skip padding
        stride = (capacity + 127) // 128 * 128 if on_gpu else capacity
        logits = ops.reference.linear(flat.float(), self.router.float())
        gates, experts, slots, (fraction, mean_prob, kept_counts) = route_tokens(logits, self.top_k, capacity,
                                                                               self.normalize_gates, stride)
        self.last_aux_loss = self.aux_loss_coef * self.num_experts * torch.sum(fraction.detach() * mean_prob)
        kept = slots >= 0
        self.last_dropped_fraction = float(1.0 - kept.float().mean()) if not x.requires_grad else None
        exchange = getattr(self.ep, "exchange", None) if self.ep is not None else None
        if exchange is not None and on_gpu:
            return self._forward_fused(flat, gates, slots, kept_counts, stride, exchange).reshape(shape)
        capacity = stride          # buffer rows per expert from here on

        # dispatch: row s of the buffer holds the token assigned to slot s (zeros where unused)
        token_of = torch.arange(tokens, device=x.device)[:, None].expand(-1, self.top_k)[kept]
        slot_of = slots[kept]
        buffer = flat.new_zeros(self.num_experts * capacity, dim).index_copy(0, slot_of, flat[token_of])
        ep_size = self.ep.size if self.ep is not None else 1
        if ep_size > 1:
            # [dst rank, local expert, C, D] -> [src rank, local expert, C, D]
            buffer = _AllToAll.apply(buffer, self.ep.group)
            grouped = buffer.reshape(ep_size, self.num_local, capacity, dim).transpose(0, 1)
            grouped = grouped.reshape(self.num_local, ep_size * capacity, dim)
        else:
            grouped = buffer.reshape(self.num_local, capacity, dim)
        result = self.experts(grouped)
        if ep_size > 1:
            result = result.reshape(self.num_local, ep_size, capacity, dim).transpose(0, 1).contiguous()
            result = _AllToAll.apply(result.reshape(-1, dim), self.ep.group)
        result = result.reshape(self.num_experts * capacity, dim)

        # combine: gate-weighted sum of each token's kept expert outputs (deterministic, slot order)
        weights = gates[kept].to(result.dtype)[:, None]
        combined = torch.zeros_like(flat).index_add(0, token_of, result[slot_of] * weights)
        if self.shared is not None:
            combined = combined + self.shared(flat)
        return combined.reshape(shape)
