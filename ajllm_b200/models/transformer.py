"""Decoder-only Transformer language model (dense or mixture-of-experts).

Architecture options, block math and checkpoint key names follow the reference
(``ajllm/modeling/transformer.py:13-126``): pre-norm ``h = x + Attn(N1 x); y = h + FFN(N2 h)`` or
post-norm ``h = N1(x + Attn x); y = N2(h + FFN h)``; RoPE / learned / no positions; RMSNorm or none;
SwiGLU or SiLU FFN; tied or untied head; ``final_norm`` only with pre-norm. Extensions: grouped KV
heads, MoE feed-forward, tensor/expert parallel shards.

Internally the residual stream is ``[tokens, d_model]`` (this rank's tokens under tensor parallelism)
and, in the pre-norm RMSNorm configuration, each residual add is fused with the norm that follows it.
"""

from __future__ import annotations

import torch
from torch import nn

from ajllm_b200 import ops
from ajllm_b200.models.attention import SelfAttention
from ajllm_b200.models.feed_forward import make_feed_forward
from ajllm_b200.models.layers import Embedding, InitSpec, Linear, make_norm
from ajllm_b200.models.moe import MoEFeedForward


class TransformerBlock(nn.Module):
    def __init__(self, d_model: int, num_heads: int, num_kv_heads: int | None, d_ff: int, context_length: int,
                 position_encoding: str, rope_theta: float, normalization: str, norm_placement: str,
                 feed_forward: str, moe: dict | None = None, init: InitSpec = InitSpec(),
                 tp=None, ep=None, norm_epsilon: float = 1e-5, cp=None) -> None:
        super().__init__()
        if norm_placement not in {"pre", "post"}:
            raise ValueError("normalization.placement must be 'pre' or 'post'")
        self.norm_placement = norm_placement
        self.norm1 = make_norm(normalization, d_model, norm_epsilon)
        self.norm2 = make_norm(normalization, d_model, norm_epsilon)
        self.attention = SelfAttention(d_model, num_heads, num_kv_heads, context_length, position_encoding,
                                       rope_theta, init, tp, cp)
        if moe:
            self.feed_forward = MoEFeedForward(d_model, moe, init, ep)
        else:
            self.feed_forward = make_feed_forward(feed_forward, d_model, d_ff, init, tp)

    def forward_prenorm(self, stream: torch.Tensor, pending: torch.Tensor | None, batch_shape):
        """``stream + pending`` is the block input; returns the new ``(stream, pending)`` pair so the
        caller (or the next block) can fuse the last residual add with its norm."""
        stream, normed = self.norm1.add_and_norm(stream, pending)
        attended = self.attention(normed, batch_shape)
        stream, normed = self.norm2.add_and_norm(stream, attended)
        return stream, self.feed_forward(normed)

    def forward_postnorm(self, x: torch.Tensor, batch_shape) -> torch.Tensor:
        hidden = self.norm1(x + self.attention(x, batch_shape))
        return self.norm2(hidden + self.feed_forward(hidden))


class TransformerLM(nn.Module):
    def __init__(self, vocab_size: int, context_length: int, d_model: int, num_layers: int, num_heads: int,
                 d_ff: int, num_kv_heads: int | None = None, position_encoding: str = "rope",
                 rope_theta: float = 10_000.0, normalization: str = "rmsnorm", norm_placement: str = "pre",
                 feed_forward: str = "swiglu", tie_embeddings: bool = False, moe: dict | None = None,
                 init: InitSpec = InitSpec(), tp=None, ep=None, norm_epsilon: float = 1e-5,
                 activation_checkpointing: str = "none", cp=None) -> None:
        super().__init__()
        if position_encoding not in {"rope", "none", "learned"}:
            raise ValueError("position encoding must be rope, none, or learned")
        self.vocab_size, self.context_length, self.d_model = vocab_size, context_length, d_model
        self.num_layers, self.num_heads, self.d_ff = num_layers, num_heads, d_ff
        self.num_kv_heads = num_kv_heads or num_heads
        self.position_encoding, self.normalization = position_encoding, normalization
        self.norm_placement, self.feed_forward_type = norm_placement, feed_forward
        self.tie_embeddings, self.moe = tie_embeddings, moe
        self.rope_theta = rope_theta
        self.tp, self.ep = tp, ep
        self.cp = cp if (cp is not None and cp.size > 1) else None
        self.activation_checkpointing = activation_checkpointing

        self.token_embeddings = Embedding(vocab_size, d_model, init)
        self.position_embeddings = Embedding(context_length, d_model, init) if position_encoding == "learned" else None
        self.layers = nn.ModuleList([
            TransformerBlock(d_model, num_heads, num_kv_heads, d_ff, context_length, position_encoding, rope_theta,
                             normalization, norm_placement, feed_forward, moe, init, tp, ep, norm_epsilon, cp)
            for _ in range(num_layers)
        ])
        self.final_norm = make_norm(normalization if norm_placement == "pre" else "none", d_model, norm_epsilon)
        self.lm_head = None if tie_embeddings else Linear(d_model, vocab_size, init)

    # ------------------------------------------------------------------ pieces
    @property
    def head_weight(self) -> torch.Tensor:
        return self.token_embeddings.weight if self.tie_embeddings else self.lm_head.weight

    def _local_tokens(self, flat: torch.Tensor) -> torch.Tensor:
        if self.tp is not None and self.tp.size > 1:
            return self.tp.local_rows(flat)
        return flat

    def _local_ids(self, per_token: torch.Tensor) -> torch.Tensor:
        """This rank's tokens of a ``[B, T]`` tensor, flattened: a slice of every sequence under context parallelism,
        a slice of the flattened rows under tensor parallelism."""
        if self.cp is not None:
            return self.cp.local_sequence(per_token, 1).reshape(-1)
        return self._local_tokens(per_token.reshape(-1))

    def hidden_states(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Final-norm output for this rank's tokens, ``[local_tokens, d_model]``."""
        B, T = token_ids.shape
        if T > self.context_length:
            raise ValueError(f"Input length {T} exceeds context length {self.context_length}")
        ids = self._local_ids(token_ids)
        stream = self.token_embeddings(ids)
        if self.position_embeddings is not None:
            positions = torch.arange(T, device=token_ids.device).repeat(B, 1)
            stream = stream + self.position_embeddings(self._local_ids(positions))
        shape = (B, T)
        if self.norm_placement == "pre":
            pending = None
            for layer in self.layers:
                if self.activation_checkpointing == "layer" and torch.is_grad_enabled():
                    from torch.utils.checkpoint import checkpoint
                    stream, pending = checkpoint(layer.forward_prenorm, stream, pending, shape, use_reentrant=False)
                else:
                    stream, pending = layer.forward_prenorm(stream, pending, shape)
            return self.final_norm.add_and_norm(stream, pending)[1]
        for layer in self.layers:
            stream = layer.forward_postnorm(stream, shape)
        return stream

    # ------------------------------------------------------------------ several micro-batches in flight
    @property
    def interleave(self) -> int:
        """Micro-batches that :meth:`loss_interleaved` runs side by side (1: the feature is off)."""
        if self.moe or self.norm_placement != "pre" or self.activation_checkpointing != "none" or self.cp is not None:
            return 1
        return int(getattr(self.tp, "interleave", 1)) if self.tp is not None else int(getattr(self, "_interleave", 1))

    @property
    def overlap_description(self) -> str | None:
        if self.interleave > 1:
            return (f"{self.interleave} micro-batches in flight on streams of their own; fused projections limited to the "
                    "SM share their NVLink transfer can feed; weight gradients on a side stream")
        return None

    def _microbatch_streams(self, count: int, device) -> list:
        streams = getattr(self, "_mb_streams", None)
        if streams is None or len(streams) < count:
            from ajllm_b200.ops import functional
            # micro-batch streams outrank the weight-gradient stream: when SMs free up, the critical path goes first
            streams = [torch.cuda.Stream(device=device, priority=-1) for _ in range(count)]
            self._mb_streams = streams
            if functional.wgrad_stream() is None:
                functional.set_wgrad_stream(torch.cuda.Stream(device=device))
        return streams[:count]

    def loss_interleaved(self, batches: list[tuple[torch.Tensor, torch.Tensor]], loss_scale: float = 1.0) -> list[torch.Tensor]:
        """:meth:`loss` of several micro-batches whose kernels are issued block by block in turn, each micro-batch on
        a stream of its own (and, under tensor parallelism, with its own fused-communication context), so that one
        micro-batch's link-bound projections overlap the other's attention and pointwise work. Backpropagate all
        returned losses in ONE ``torch.autograd.backward(losses)`` call (autograd then alternates between the
        micro-batches in the same way, each on its forward stream), then call :meth:`join_streams`.

        In-place gradient accumulations that are not atomic are kept apart: weight gradients all go through one side
        stream (:func:`ajllm_b200.ops.functional.wgrad_accumulate`), and the LM head's loss-and-gradient chunks of one
        micro-batch start only when the previous micro-batch's are done."""
        count = len(batches)
        device = batches[0][0].device
        main = torch.cuda.current_stream()
        streams = self._microbatch_streams(count, device)
        from ajllm_b200.ops import functional
        functional.wgrad_stream().wait_stream(main)
        states, shapes = [], []
        for index, (token_ids, _) in enumerate(batches):
            B, T = token_ids.shape
            if T > self.context_length:
                raise ValueError(f"Input length {T} exceeds context length {self.context_length}")
            streams[index].wait_stream(main)
            with torch.cuda.stream(streams[index]):
                stream = self.token_embeddings(self._local_tokens(token_ids.reshape(-1)))
                if self.position_embeddings is not None:
                    positions = torch.arange(T, device=device).repeat(B)
                    stream = stream + self.position_embeddings(self._local_tokens(positions))
            states.append((stream, None))
            shapes.append((B, T))
        for layer in self.layers:
            for index in range(count):
                if self.tp is not None:
                    self.tp.select(index)
                with torch.cuda.stream(streams[index]):
                    states[index] = layer.forward_prenorm(states[index][0], states[index][1], shapes[index])
        losses = []
        head_done = None
        share = float(getattr(self, "data_parallel_share", 1.0))
        if self.tp is not None and self.tp.size > 1:
            share = share / self.tp.size
        for index, (_, targets) in enumerate(batches):
            with torch.cuda.stream(streams[index]):
                hidden = self.final_norm.add_and_norm(states[index][0], states[index][1])[1]
                if head_done is not None:
                    streams[index].wait_event(head_done)
                local_targets = self._local_tokens(targets.reshape(-1))
                losses.append(ops.linear_cross_entropy(hidden, self.head_weight, local_targets, loss_scale) * share)
                head_done = streams[index].record_event()
        if self.tp is not None:
            self.tp.select(0)
        return losses

    def join_streams(self) -> None:
        """The current stream waits for the micro-batch streams and for the weight-gradient stream."""
        from ajllm_b200.ops import functional
        main = torch.cuda.current_stream()
        for stream in getattr(self, "_mb_streams", None) or []:
            main.wait_stream(stream)
        functional.join_wgrad_stream()

    def aux_loss(self) -> torch.Tensor | None:
        terms = [layer.feed_forward.last_aux_loss for layer in self.layers
                 if isinstance(layer.feed_forward, MoEFeedForward) and layer.feed_forward.last_aux_loss is not None]
        return sum(terms) if terms else None

    # ------------------------------------------------------------------ public
    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        """Logits ``[B, T, vocab]`` (all tokens on every rank)."""
        B, T = token_ids.shape
        logits = ops.linear(self.hidden_states(token_ids), self.head_weight)
        if self.tp is not None and self.tp.size > 1:
            logits = self.tp.all_gather_cat(logits, 0, differentiable=True)
        if self.cp is not None:
            local = logits.reshape(B, T // self.cp.size, self.vocab_size)
            return self.cp.all_gather_cat(local, 1, differentiable=True)
        return logits.reshape(B, T, self.vocab_size)

    def loss(self, token_ids: torch.Tensor, targets: torch.Tensor, loss_scale: float = 1.0) -> torch.Tensor:
        """Mean next-token cross-entropy without materialising the logits.

        Under tensor parallelism each rank scores its own tokens; the returned value is that rank's
        share ``sum_local / N_global`` (sum over ranks = global mean), which is also the quantity whose
        gradient the sharded backward needs.
        """
        hidden = self.hidden_states(token_ids)
        local_targets = self._local_ids(targets)
        # replicated data parallelism sets `data_parallel_share = 1 / dp` so that gradients and losses of the
        # replicas add up to those of the global batch with plain sums
        share = float(getattr(self, "data_parallel_share", 1.0))
        if self.tp is not None and self.tp.size > 1:
            share = share / self.tp.size
        if self.cp is not None:
            share = share / self.cp.size
        loss = ops.linear_cross_entropy(hidden, self.head_weight, local_targets, loss_scale) * share
        aux = self.aux_loss()
        if aux is not None:
            loss = loss + aux * (share * loss_scale if loss_scale != 1.0 else share)
        return loss
