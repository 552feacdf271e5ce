"""Position-wise feed-forward networks.

``SwiGLU(x) = W2(silu(W1 x) * W3 x)`` and ``SiLU-FFN(x) = W2 silu(W1 x)`` as in the reference
(``ajllm/modeling/activations.py:15-45``). W1 and W3 are stored as one ``[2F, D]`` matrix with rows
interleaved (row ``2j`` = W1 row ``j``, row ``2j+1`` = W3 row ``j``), so one GEMM yields gate/up pairs in
adjacent columns. ``state_dict`` exposes ``w1.weight`` / ``w3.weight`` / ``w2.weight``.
"""

from __future__ import annotations

import torch
from torch import nn

from ajllm_b200 import ops
from ajllm_b200.models.layers import InitSpec, init_matrix_


def interleave_rows(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return torch.stack((gate, up), dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()


def deinterleave_rows(packed: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    pairs = packed.reshape(packed.shape[0] // 2, 2, packed.shape[1])
    return pairs[:, 0], pairs[:, 1]


class SwiGLU(nn.Module):
    def __init__(self, d_model: int, d_ff: int, init: InitSpec = InitSpec(), tp=None) -> None:
        super().__init__()
        self.d_model, self.total_d_ff, self.tp = d_model, d_ff, tp
        tp_size = tp.size if tp is not None else 1
        if d_ff % tp_size:
            raise ValueError("tensor parallel size must divide d_ff")
        self.d_ff = d_ff // tp_size
        w1, w2, w3 = torch.empty(d_ff, d_model), torch.empty(d_model, d_ff), torch.empty(d_ff, d_model)
        # reference construction order: w1, w2, w3
        init_matrix_(w1, d_model, d_ff, init)
        init_matrix_(w2, d_ff, d_model, init)
        init_matrix_(w3, d_model, d_ff, init)
        self.w13 = nn.Parameter(interleave_rows(w1[self._rows()], w3[self._rows()]))
        self.w2 = nn.Parameter(w2[:, self._rows()].contiguous())
        self._register_state_dict_hook(self._split_on_save)
        self._register_load_state_dict_pre_hook(self._merge_on_load)

    def _rows(self) -> slice:
        rank = self.tp.rank if self.tp is not None else 0
        return slice(rank * self.d_ff, (rank + 1) * self.d_ff)

    def _gather_full(self, local, dim):
        if self.tp is None or self.tp.size == 1:
            return local
        return self.tp.all_gather_cat(local.contiguous(), dim)

    def _split_on_save(self, module, state, prefix, local_metadata):
        gate, up = deinterleave_rows(state.pop(prefix + "w13"))
        down = state.pop(prefix + "w2")
        state[prefix + "w1.weight"] = self._gather_full(gate, 0).clone()
        state[prefix + "w2.weight"] = self._gather_full(down, 1).clone()
        state[prefix + "w3.weight"] = self._gather_full(up, 0).clone()
        return state

    def _merge_on_load(self, state, prefix, *unused):
        k1, k2, k3 = (prefix + f"w{i}.weight" for i in (1, 2, 3))
        if k1 in state and k3 in state:
            state[prefix + "w13"] = interleave_rows(state.pop(k1)[self._rows()], state.pop(k3)[self._rows()])
        if k2 in state:
            state[prefix + "w2"] = state.pop(k2)[:, self._rows()].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            return self.tp.swiglu_ffn(x, self.w13, self.w2)
        return ops.swiglu_ffn(x, self.w13, self.w2)


class SiLUFeedForward(nn.Module):
    def __init__(self, d_model: int, d_ff: int, init: InitSpec = InitSpec(), tp=None) -> None:
        super().__init__()
        self.tp = tp
        tp_size = tp.size if tp is not None else 1
        if d_ff % tp_size:
            raise ValueError("tensor parallel size must divide d_ff")
        self.d_ff = d_ff // tp_size
        rank = tp.rank if tp is not None else 0
        rows = slice(rank * self.d_ff, (rank + 1) * self.d_ff)
        w1, w2 = torch.empty(d_ff, d_model), torch.empty(d_model, d_ff)
        init_matrix_(w1, d_model, d_ff, init)
        init_matrix_(w2, d_ff, d_model, init)
        self._rows_slice = rows
        self.w1 = nn.Parameter(w1[rows].contiguous())
        self.w2 = nn.Parameter(w2[:, rows].contiguous())
        self._register_state_dict_hook(self._rename_on_save)
        self._register_load_state_dict_pre_hook(self._rename_on_load)

    def _gather_full(self, local, dim):
        if self.tp is None or self.tp.size == 1:
            return local
        return self.tp.all_gather_cat(local.contiguous(), dim)

    def _rename_on_save(self, module, state, prefix, local_metadata):
        state[prefix + "w1.weight"] = self._gather_full(state.pop(prefix + "w1"), 0).clone()
        state[prefix + "w2.weight"] = self._gather_full(state.pop(prefix + "w2"), 1).clone()
        return state

    def _rename_on_load(self, state, prefix, *unused):
        if prefix + "w1.weight" in state:
            state[prefix + "w1"] = state.pop(prefix + "w1.weight")[self._rows_slice].contiguous()
        if prefix + "w2.weight" in state:
            state[prefix + "w2"] = state.pop(prefix + "w2.weight")[:, self._rows_slice].contiguous()

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            return self.tp.linear_scatter(ops.silu(self.tp.gather_linear(x, self.w1)), self.w2)
        return ops.linear(ops.silu(ops.linear(x, self.w1)), self.w2)


def make_feed_forward(kind: str, d_model: int, d_ff: int, init: InitSpec = InitSpec(), tp=None) -> nn.Module:
    if kind == "swiglu":
        return SwiGLU(d_model, d_ff, init, tp)
    if kind == "silu":
        return SiLUFeedForward(d_model, d_ff, init, tp)
    raise ValueError(f"Unsupported feed-forward type: {kind}")
