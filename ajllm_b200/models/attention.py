"""Causal self-attention with grouped KV heads and interleaved RoPE.

The reference has four ``[d_model, d_model]`` projections and multi-head attention only
(``ajllm/modeling/attention.py:63-120``). Here the q/k/v projections are stored as one
``[(Hq + 2 Hkv) * hd, d_model]`` matrix so they run as a single GEMM whose packed output the attention
kernel reads in place; ``state_dict`` still exposes ``q_proj.weight`` / ``k_proj.weight`` /
``v_proj.weight`` (and loads them), so checkpoints keep the reference's key names. Under tensor
parallelism a rank holds ``Hq / tp`` query heads and ``Hkv / tp`` KV heads (column-parallel qkv,
row-parallel output projection) and activations between blocks are sharded by token.
"""

from __future__ import annotations

import torch
from torch import nn

from ajllm_b200 import ops
from ajllm_b200.models.layers import InitSpec, init_matrix_
from ajllm_b200.ops import reference


class SelfAttention(nn.Module):
    def __init__(self, d_model: int, num_heads: int, num_kv_heads: int | None, context_length: int,
                 position_encoding: str, rope_theta: float, init: InitSpec = InitSpec(), tp=None, cp=None) -> None:
        super().__init__()
        if d_model % num_heads:
            raise ValueError("d_model must be divisible by num_heads")
        num_kv_heads = num_kv_heads or num_heads
        if num_heads % num_kv_heads:
            raise ValueError("num_kv_heads must divide num_heads")
        self.d_model = d_model
        self.total_heads, self.total_kv_heads = num_heads, num_kv_heads
        self.head_dim = d_model // num_heads
        self.tp = tp
        self.cp = cp if (cp is not None and cp.size > 1) else None      # context parallelism: sequence split <-> head split
        if self.cp is not None:
            if tp is not None and tp.size > 1:
                raise ValueError("context parallelism and tensor parallelism are not combined")
            self.cp.check_heads(num_heads, num_kv_heads)
        self.qkv_override = None
        tp_size = tp.size if tp is not None else 1
        if num_heads % tp_size or num_kv_heads % tp_size:
            raise ValueError("tensor parallel size must divide both head counts")
        self.num_heads = num_heads // tp_size
        self.num_kv_heads = num_kv_heads // tp_size
        self.context_length = context_length
        self.use_rope = position_encoding == "rope"
        self.rope_theta = rope_theta

        hd = self.head_dim
        full_q = torch.empty(num_heads * hd, d_model)
        full_k = torch.empty(num_kv_heads * hd, d_model)
        full_v = torch.empty(num_kv_heads * hd, d_model)
        full_o = torch.empty(d_model, num_heads * hd)
        # draw in the reference's order (q, k, v, output) so equal seeds give equal MHA weights
        init_matrix_(full_q, d_model, num_heads * hd, init)
        init_matrix_(full_k, d_model, d_model if num_kv_heads == num_heads else num_kv_heads * hd, init)
        init_matrix_(full_v, d_model, d_model if num_kv_heads == num_heads else num_kv_heads * hd, init)
        init_matrix_(full_o, num_heads * hd, d_model, init)
        self.qkv_proj = nn.Parameter(self.pack_qkv(*self._shard_qkv(full_q, full_k, full_v)))
        self.output_proj = nn.Parameter(self._shard_out(full_o))
        # cos/sin tables stay fp32 whatever dtype the module is cast to (the kernels read fp32), so they
        # are cached per device instead of being registered as buffers
        self._rope_tables: dict = {}
        self._register_state_dict_hook(self._split_on_save)
        self._register_load_state_dict_pre_hook(self._merge_on_load)

    # ----- sharding helpers (identity without tensor parallelism)
    def _rank_slice(self, heads: int) -> slice:
        rank = self.tp.rank if self.tp is not None else 0
        width = heads * self.head_dim
        return slice(rank * width, (rank + 1) * width)

    def _shard_qkv(self, q, k, v):
        return q[self._rank_slice(self.num_heads)], k[self._rank_slice(self.num_kv_heads)], \
            v[self._rank_slice(self.num_kv_heads)]

    def _shard_out(self, o):
        return o[:, self._rank_slice(self.num_heads)].contiguous()

    @staticmethod
    def pack_qkv(q, k, v):
        return torch.cat((q, k, v), dim=0).contiguous()

    def unpack_qkv(self, packed):
        nq, nk = self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        return packed[:nq], packed[nq:nq + nk], packed[nq + nk:]

    # ----- reference-compatible checkpoint keys
    def _gather_full(self, local: torch.Tensor, dim: int) -> torch.Tensor:
        if self.tp is None or self.tp.size == 1:
            return local
        return self.tp.all_gather_cat(local.contiguous(), dim)

    def _split_on_save(self, module, state, prefix, local_metadata):
        packed = state.pop(prefix + "qkv_proj")
        out = state.pop(prefix + "output_proj")
        q, k, v = self.unpack_qkv(packed)
        state[prefix + "q_proj.weight"] = self._gather_full(q, 0).clone()
        state[prefix + "k_proj.weight"] = self._gather_full(k, 0).clone()
        state[prefix + "v_proj.weight"] = self._gather_full(v, 0).clone()
        state[prefix + "output_proj.weight"] = self._gather_full(out, 1).clone()
        return state

    def _merge_on_load(self, state, prefix, *unused):
        keys = [prefix + name + ".weight" for name in ("q_proj", "k_proj", "v_proj")]
        if all(key in state for key in keys):
            q, k, v = (state.pop(key) for key in keys)
            state[prefix + "qkv_proj"] = self.pack_qkv(*self._shard_qkv(q, k, v))
        key = prefix + "output_proj.weight"
        if key in state:
            state[prefix + "output_proj"] = self._shard_out(state.pop(key))

    def rope_tables(self, device) -> tuple[torch.Tensor | None, torch.Tensor | None]:
        if not self.use_rope:
            return None, None
        key = str(device)
        if key not in self._rope_tables:
            self._rope_tables[key] = reference.rope_tables(self.head_dim, self.context_length, self.rope_theta, device)
        return self._rope_tables[key]

    @property
    def rope_cos(self):
        return self.rope_tables(self.qkv_proj.device)[0]

    @property
    def rope_sin(self):
        return self.rope_tables(self.qkv_proj.device)[1]

    # ----- compute
    def project_qkv(self, x: torch.Tensor) -> torch.Tensor:
        """``x`` holds this rank's tokens; the result covers all tokens and this rank's heads."""
        if self.qkv_override is not None:         # a wrapper that produces the projection its own way (sharded weights)
            return self.qkv_override(x)
        if self.tp is not None and self.tp.size > 1:
            return self.tp.gather_linear(x, self.qkv_proj)
        return ops.linear(x, self.qkv_proj)

    def project_out(self, attended: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            return self.tp.linear_scatter(attended, self.output_proj)
        return ops.linear(attended, self.output_proj)

    def forward(self, x: torch.Tensor, batch_shape: tuple[int, int]) -> torch.Tensor:
        """``x`` is ``[local_tokens, d_model]`` (or ``[B, T, d_model]`` without TP); ``batch_shape`` is
        the global ``(B, T)`` the tokens were flattened from."""
        B, T = batch_shape
        if self.cp is not None:
            cp = self.cp
            # x holds T / cp tokens of every sequence: trade the sequence split for a head split around the kernel
            qkv = cp.to_heads(self.project_qkv(x).reshape(B, T // cp.size, -1), self.num_heads, self.num_kv_heads,
                              self.head_dim)
            attended = ops.rope_attention(qkv, self.rope_cos, self.rope_sin, self.num_heads // cp.size,
                                          self.num_kv_heads // cp.size, self.head_dim, causal=True)
            attended = cp.to_sequence(attended, self.num_heads, self.head_dim)
            return self.project_out(attended.reshape(B * (T // cp.size), -1)).reshape(x.shape)
        qkv = self.project_qkv(x).reshape(B, T, -1)
        attended = ops.rope_attention(qkv, self.rope_cos, self.rope_sin, self.num_heads, self.num_kv_heads,
                                      self.head_dim, causal=True)
        out = self.project_out(attended.reshape(B * T, -1))
        return out.reshape(x.shape)
