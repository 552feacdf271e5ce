"""Fully sharded data parallelism (ZeRO-3) with per-layer activation checkpointing.

What the reference does (``ajllm/training/distributed.py:164-379``): every Linear/Embedding weight is a
flat fp32 shard; each is all-gathered synchronously right before use (twice per step under its
"activation checkpointing", which only drops the gathered weight), gradients are reduce-scattered per
tensor in fp32, norm gains stay replicated and are all-reduced one tensor at a time, nothing overlaps.

Here the unit of sharding is a *layer*: all tensors of a unit (embeddings | one block | final norm +
head) live in one flat buffer that is split evenly over the data-parallel group, so a step needs one
all-gather per unit per pass and one reduce-scatter per unit, each a single large message, and the
next unit's gather is issued on a side stream while the current unit computes. Forward runs unit by
unit without autograd and keeps only each unit's input; backward re-gathers a unit, recomputes it
with autograd, back-propagates, and reduce-scatters that unit's fp32 gradients into the rank's
gradient shard (accumulating over micro-batches). This is real per-layer activation checkpointing:
block-internal activations never outlive their unit. Norm gains are sharded like everything else.
All shards of all units form one flat buffer per kind (master, gradient, moments, working copy), so
the global gradient norm is one reduction plus one small all-reduce and AdamW is one kernel.
Expert-parallel weights are not gathered: they stay local, and only their replicas (if the
data-parallel group is larger than the expert-parallel group) exchange gradients.

Tied embeddings are supported (the reference crashes on them, ``distributed.py:248``): the head
borrows the embedding unit's gathered weight.
"""

from __future__ import annotations

import os

from dataclasses import dataclass, field
from typing import Any

import torch
import torch.distributed as dist
from torch import nn

from ajllm_b200 import ops
from ajllm_b200.training.optim import flat_adamw, flat_sumsq

_ALIGN = 64


@dataclass
class _Unit:
    name: str
    modules: list[tuple[str, nn.Module]]          # (state-dict prefix, module)
    params: list[nn.Parameter] = field(default_factory=list)
    names: list[str] = field(default_factory=list)
    offsets: list[int] = field(default_factory=list)
    padded: int = 0                                # full flat length (multiple of world * _ALIGN)
    shard: int = 0                                 # per-rank length
    base: int = 0                                  # offset of this unit's shard in the rank-wide flat buffers


class _GatherWeightLinearFn(torch.autograd.Function):
    """``x @ W^T`` where producing the output also makes ``W`` resident: ``produce(x)`` runs the kernel that gathers
    the unit's flat parameter buffer while it multiplies (``csrc/comm_gemm.cu`` mode 3) and points the unit's
    parameters at the gathered buffer. The backward pass is the ordinary one, on the then-resident weight."""

    @staticmethod
    def forward(ctx, x, weight, produce):
        x2 = x.reshape(-1, x.shape[-1]).contiguous()
        out = produce(x2)
        ctx.save_for_backward(x2, weight)
        ctx.lead = x.shape[:-1]
        return out.view(*ctx.lead, out.shape[-1])

    @staticmethod
    def backward(ctx, grad_out):
        from ajllm_b200.ops.functional import gemm, wgrad_epilogue
        x2, weight = ctx.saved_tensors
        n, k = weight.shape
        g2 = grad_out.reshape(-1, n).to(torch.bfloat16).contiguous()
        m = g2.shape[0]
        grad_x = None
        if ctx.needs_input_grad[0]:
            grad_x = torch.empty(m, k, dtype=torch.bfloat16, device=g2.device)
            gemm(g2, weight, grad_x, m, k, n, b_mn_major=True)
            grad_x = grad_x.view(*ctx.lead, k)
        grad_w = None
        main = getattr(weight, "main_grad", None)
        if main is not None:
            gemm(g2, x2, main, n, k, m, a_mn_major=True, b_mn_major=True, epilogue=wgrad_epilogue())
            weight.main_grad_written = True
        else:
            grad_w = torch.empty(n, k, dtype=torch.bfloat16, device=g2.device)
            gemm(g2, x2, grad_w, n, k, m, a_mn_major=True, b_mn_major=True)
        return grad_x, grad_w, None


class ShardedOptimizer:
    """AdamW over this rank's shards; same surface as :class:`~ajllm_b200.training.optim.FlatAdamW`."""

    def __init__(self, owner: "ShardedDataParallel", learning_rate, betas, epsilon, weight_decay) -> None:
        self.owner = owner
        self.param_groups = [{"lr": learning_rate, "betas": tuple(betas), "eps": epsilon, "weight_decay": weight_decay}]
        self.step_count = 0

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.owner.join_reductions()
        self.owner.grad.zero_()
        if self.owner.local_grad is not None:
            self.owner.local_grad.zero_()

    @torch.no_grad()
    def step(self, max_norm: float = 0.0) -> torch.Tensor:
        o = self.owner
        o.join_reductions()
        # the fused reduce-scatter left per-CTA sums of squares of every unit's (fully accumulated) shard
        sumsq = o._sumsq_partials.sum().reshape(1) if o.fused_reduce is not None else flat_sumsq(o.grad).clone()
        if o.local_grad is not None:
            if o.replica_group is not None:
                dist.all_reduce(o.local_grad, op=dist.ReduceOp.SUM, group=o.replica_group)
            sumsq += flat_sumsq(o.local_grad) / o.replicas
        dist.all_reduce(sumsq, op=dist.ReduceOp.SUM, group=o.group)
        self.step_count += 1
        g = self.param_groups[0]
        b1, b2 = g["betas"]
        flat_adamw(o.master, o.grad, o.m, o.v, None if o.master is o.working else o.working, self.step_count,
                   g["lr"], b1, b2, g["eps"], g["weight_decay"], sumsq, max_norm)
        if o.local_grad is not None:
            flat_adamw(o.local_master, o.local_grad, o.local_m, o.local_v,
                       None if o.local_master is o.local_working else o.local_working, self.step_count,
                       g["lr"], b1, b2, g["eps"], g["weight_decay"], sumsq, max_norm)
        o.refresh_norm_cache()
        return sumsq.sqrt()

    def state_dict(self) -> dict[str, Any]:
        o = self.owner
        first, second = o.export_named(o.m, o.local_m), o.export_named(o.v, o.local_v)
        names = list(first)
        state = {i: {"step": self.step_count, "first_moment": first[n], "second_moment": second[n]}
                 for i, n in enumerate(names)} if self.step_count else {}
        group = dict(self.param_groups[0])
        group["params"] = list(range(len(names)))
        out = {"state": state, "param_groups": [group], "param_names": names}
        if o.master is not o.working:
            out["master_weights"] = o.export_named(o.master, o.local_master)
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        o = self.owner
        group = state_dict["param_groups"][0]
        for key in ("lr", "betas", "eps", "weight_decay"):
            if key in group:
                self.param_groups[0][key] = tuple(group[key]) if key == "betas" else group[key]
        state = state_dict.get("state") or {}
        names = state_dict.get("param_names")
        if state and names:
            entries = [state[k] for k in sorted(state, key=int)]
            self.step_count = int(entries[0]["step"])
            o.import_named({n: e["first_moment"] for n, e in zip(names, entries)}, o.m, o.local_m)
            o.import_named({n: e["second_moment"] for n, e in zip(names, entries)}, o.v, o.local_v)
        if o.master is not o.working:
            masters = state_dict.get("master_weights")
            if masters is not None:
                o.import_named(masters, o.master, o.local_master)
            else:
                o.master.copy_(o.working.float())
                if o.local_master is not None:
                    o.local_master.copy_(o.local_working.float())


class ShardedDataParallel(nn.Module):
    def __init__(self, module, group, checkpoint_layers: bool = True, learning_rate: float = 1e-3,
                 betas=(0.9, 0.95), epsilon: float = 1e-8, weight_decay: float = 0.0,
                 replica_group=None, replicas: int = 1, prefetch: bool = True, fused_reduce: bool | None = None,
                 fused_gather: bool | None = None) -> None:
        super().__init__()
        if module.norm_placement != "pre":
            raise ValueError("sharded training supports pre-norm models")
        self.module = module
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.replica_group, self.replicas = replica_group, replicas
        self.checkpoint_layers = checkpoint_layers
        first = next(module.parameters())
        self.device, self.dtype = first.device, first.dtype
        self.prefetch = prefetch and self.device.type == "cuda"
        ep = getattr(module, "ep", None)
        self._ep_active = ep is not None and ep.size > 1

        self.units = self._make_units()
        cursor = 0
        for unit in self.units:
            unit.base = cursor
            cursor += unit.shard
        self.total_shard = cursor
        dev = self.device
        self.working = torch.zeros(cursor, dtype=self.dtype, device=dev)
        self.grad = torch.zeros(cursor, dtype=torch.float32, device=dev)
        self.m = torch.zeros(cursor, dtype=torch.float32, device=dev)
        self.v = torch.zeros(cursor, dtype=torch.float32, device=dev)
        largest = max(u.padded for u in self.units)
        self._full = [torch.empty(largest, dtype=self.dtype, device=dev) for _ in range(2 if self.prefetch else 1)]
        # Gradient reduce-scatter: one fused kernel over symmetric memory (pull + add + shard accumulation +
        # partial sums of squares) on GPUs, NCCL reduce_scatter + add_ elsewhere or when switched off.
        if fused_reduce is None:
            fused_reduce = dev.type == "cuda" and 1 < self.world <= 8 and os.environ.get("AJB_FUSED_FSDP", "1") != "0"
        self.fused_reduce = None
        # With the fused kernel the reduction of a unit runs on a stream of its own while the next unit already
        # back-propagates into a second full-gradient buffer (AJB_FSDP_OVERLAP_REDUCE=0: one buffer, in stream order).
        self._reducers: list = []
        self._reduce_stream = None
        self._reduce_events: list = [None, None]
        self._grad_slot = 0
        if fused_reduce:
            from ajllm_b200.parallel.grad_reduce import FusedGradReduce
            overlap = os.environ.get("AJB_FSDP_OVERLAP_REDUCE", "1") != "0"
            self._reducers = [FusedGradReduce(group, dev, largest) for _ in range(2 if overlap else 1)]
            self.fused_reduce = self._reducers[0]
            self._full_grad = self.fused_reduce.buffer
            self._sumsq_partials = torch.zeros(len(self.units), FusedGradReduce.CTAS, dtype=torch.float32, device=dev)
            if overlap:
                self._reduce_stream = torch.cuda.Stream(device=dev)
        else:
            self._full_grad = torch.zeros(largest, dtype=torch.float32, device=dev)
        # Parameter all-gather of a block fused into its first GEMM (the QKV projection): opt-in, bf16 on GPUs.
        # Needs the block's first norm gain before the block's parameters arrive: every rank keeps a copy of those.
        if fused_gather is None:
            fused_gather = os.environ.get("AJB_FUSED_FSDP_GATHER", "0") == "1"
        self.fused_gather = None
        self._norm_cache: dict[int, torch.Tensor] = {}
        if fused_gather and dev.type == "cuda" and self.dtype == torch.bfloat16 and 1 < self.world <= 8:
            from ajllm_b200.parallel.fused import FusedTensorParallel
            self.fused_gather = FusedTensorParallel(group, dev)
        self._resident: dict[int, int] = {}          # unit index -> slot of self._full holding it
        self._gather_events: dict[int, Any] = {}
        self._side = torch.cuda.Stream(device=dev) if self.prefetch else None
        with torch.no_grad():
            self._scatter_initial_weights()
        self.master = self.working if self.dtype == torch.float32 else self.working.float()
        self._setup_local_params()
        self.optimizer = ShardedOptimizer(self, learning_rate, betas, epsilon, weight_decay)
        if self.fused_gather is not None:
            self.refresh_norm_cache()

    # ------------------------------------------------------------------ construction
    def _is_local(self, name: str) -> bool:
        return self._ep_active and ".experts." in name

    def _make_units(self) -> list[_Unit]:
        m = self.module
        units = [_Unit("embeddings", [("token_embeddings.", m.token_embeddings)])]
        if m.position_embeddings is not None:
            units[0].modules.append(("position_embeddings.", m.position_embeddings))
        for i, layer in enumerate(m.layers):
            units.append(_Unit(f"layer{i}", [(f"layers.{i}.", layer)]))
        tail = _Unit("head", [("final_norm.", m.final_norm)])
        if m.lm_head is not None:
            tail.modules.append(("lm_head.", m.lm_head))
        units.append(tail)
        step = self.world * _ALIGN
        for unit in units:
            cursor = 0
            for prefix, mod in unit.modules:
                for name, p in mod.named_parameters():
                    if self._is_local(prefix + name):
                        continue
                    p._full_shape = p.shape
                    unit.params.append(p)
                    unit.names.append(prefix + name)
                    unit.offsets.append(cursor)
                    cursor += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
            unit.padded = max(step, (cursor + step - 1) // step * step)
            unit.shard = unit.padded // self.world
        return units

    def _scatter_initial_weights(self) -> None:
        """Rank 0's initial values become everyone's (one broadcast per unit), then each rank keeps its slice."""
        for unit in self.units:
            full = self._full[0][:unit.padded]
            full.zero_()
            for p, off in zip(unit.params, unit.offsets):
                full[off:off + p._full_shape.numel()].copy_(p.data.reshape(-1))
            src = dist.get_global_rank(self.group, 0) if hasattr(dist, "get_global_rank") else 0
            dist.broadcast(full, src=src, group=self.group)
            self.working[unit.base:unit.base + unit.shard].copy_(full[self.rank * unit.shard:(self.rank + 1) * unit.shard])
            for p in unit.params:
                p.data = torch.empty(0, dtype=self.dtype, device=self.device)

    def _setup_local_params(self) -> None:
        named = [(n, p) for n, p in self.module.named_parameters() if self._is_local(n)]
        self.local_named = named
        self.local_grad = self.local_master = self.local_working = self.local_m = self.local_v = None
        if not named:
            return
        offsets, cursor = [], 0
        for _, p in named:
            offsets.append(cursor)
            cursor += (p.numel() + _ALIGN - 1) // _ALIGN * _ALIGN
        self.local_offsets = offsets
        dev = self.device
        self.local_working = torch.zeros(cursor, dtype=self.dtype, device=dev)
        self.local_grad = torch.zeros(cursor, dtype=torch.float32, device=dev)
        self.local_m, self.local_v = torch.zeros_like(self.local_grad), torch.zeros_like(self.local_grad)
        for (_, p), off in zip(named, offsets):
            view = self.local_working[off:off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.local_grad[off:off + p.numel()].view(p.shape)
        self.local_master = self.local_working if self.dtype == torch.float32 else self.local_working.float()

    # ------------------------------------------------------------------ gather / release / reduce
    def _issue_gather(self, index: int) -> None:
        if index in self._resident or not 0 <= index < len(self.units):
            return
        unit = self.units[index]
        busy = set(self._resident.values())
        slot = next((s for s in range(len(self._full)) if s not in busy), None)
        if slot is None:
            return
        full = self._full[slot][:unit.padded]
        shard = self.working[unit.base:unit.base + unit.shard]
        if self._side is not None:
            self._side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(self._side):
                dist.all_gather_into_tensor(full, shard, group=self.group)
                event = torch.cuda.Event()
                event.record(self._side)
            self._gather_events[index] = event
        else:
            dist.all_gather_into_tensor(full, shard, group=self.group)
        self._resident[index] = slot

    def _acquire(self, index: int, prefetch_next: int | None = None) -> None:
        """Make unit ``index`` usable on the current stream and start fetching ``prefetch_next``."""
        self._issue_gather(index)
        if index not in self._resident:
            raise RuntimeError("no free gather buffer: a unit was not released")
        event = self._gather_events.pop(index, None)
        if event is not None:
            torch.cuda.current_stream().wait_event(event)
        unit = self.units[index]
        full = self._full[self._resident[index]]
        for p, off in zip(unit.params, unit.offsets):
            p.data = full[off:off + p._full_shape.numel()].view(p._full_shape)
        if prefetch_next is not None and self.prefetch:
            self._issue_gather(prefetch_next)

    def _release(self, index: int) -> None:
        unit = self.units[index]
        for p in unit.params:
            p.data = torch.empty(0, dtype=self.dtype, device=self.device)
        self._resident.pop(index, None)

    def join_reductions(self) -> None:
        """The current stream waits for the gradient reductions still running on their own stream."""
        if self._reduce_stream is not None:
            torch.cuda.current_stream().wait_stream(self._reduce_stream)

    def _attach_grad_views(self, unit: _Unit) -> None:
        if self._reduce_stream is not None:
            # alternate between the two full-gradient buffers; the one taken now was last reduced two units ago
            self._grad_slot ^= 1
            self.fused_reduce = self._reducers[self._grad_slot]
            self._full_grad = self.fused_reduce.buffer
            pending = self._reduce_events[self._grad_slot]
            if pending is not None:
                torch.cuda.current_stream().wait_event(pending)
        self._full_grad[:unit.padded].zero_()
        for p, off in zip(unit.params, unit.offsets):
            p.main_grad = self._full_grad[off:off + p._full_shape.numel()].view(p._full_shape)
            p.main_grad_written = False
            p.grad = None

    def _reduce_unit_grads(self, index: int) -> None:
        unit = self.units[index]
        for p in unit.params:
            if p.grad is not None:                                   # ops that went through autograd
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None
        for _, p in self.local_named:                                # expert-parallel tensors stay local
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None
        if self.fused_reduce is not None and self._reduce_stream is not None:
            side = self._reduce_stream
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                self.fused_reduce.reduce_into(self.grad[unit.base:unit.base + unit.shard], unit.shard, accumulate=True,
                                              sumsq_partials=self._sumsq_partials[index])
                self._reduce_events[self._grad_slot] = side.record_event()
        elif self.fused_reduce is not None:
            self.fused_reduce.reduce_into(self.grad[unit.base:unit.base + unit.shard], unit.shard, accumulate=True,
                                          sumsq_partials=self._sumsq_partials[index])
        else:
            out = torch.empty(unit.shard, dtype=torch.float32, device=self.device)
            dist.reduce_scatter_tensor(out, self._full_grad[:unit.padded], op=dist.ReduceOp.SUM, group=self.group)
            self.grad[unit.base:unit.base + unit.shard].add_(out)
        for p in unit.params:
            p.main_grad = None

    # ------------------------------------------------------------------ gather fused into the first GEMM of a block
    def refresh_norm_cache(self) -> None:
        """Copies of every block's first norm gain on every rank (one small broadcast; after each optimizer step)."""
        if self.fused_gather is None:
            return
        layers = list(self.module.layers)
        d = self.module.d_model
        packed = torch.empty(len(layers), d, dtype=self.dtype, device=self.device)
        for i, layer in enumerate(layers, start=1):
            unit = self.units[i]
            off = self._offset_of(unit, layer.norm1.weight)
            if off + d > unit.shard:
                raise ValueError("a block's first norm gain must lie inside the first rank's slice of its unit")
            if self.rank == 0:
                packed[i - 1].copy_(self.working[unit.base + off:unit.base + off + d])
        src = dist.get_global_rank(self.group, 0) if hasattr(dist, "get_global_rank") else 0
        dist.broadcast(packed, src=src, group=self.group)
        self._norm_cache = {i: packed[i - 1] for i in range(1, len(layers) + 1)}

    @staticmethod
    def _offset_of(unit: _Unit, param) -> int:
        """Offset of ``param`` in its unit's flat buffer (identity search: ``==`` on tensors is element-wise)."""
        return next(off for p, off in zip(unit.params, unit.offsets) if p is param)

    def _make_resident(self, index: int, slot: int) -> None:
        unit = self.units[index]
        full = self._full[slot]
        for p, off in zip(unit.params, unit.offsets):
            p.data = full[off:off + p._full_shape.numel()].view(p._full_shape)
        self._resident[index] = slot

    def _run_block(self, index: int, layer, stream, pending, shape, prefetch_next: int | None):
        """Forward of block ``index`` (unit number). Default: make the unit resident (NCCL all-gather, usually
        prefetched one unit ahead), then run the block. With the fused gather and a unit that is not resident
        yet, the QKV projection itself gathers the unit (its first norm runs on the cached gain)."""
        attn = layer.attention
        fusable = (self.fused_gather is not None and index not in self._resident and index in self._norm_cache
                   and stream.dim() == 2 and stream.shape[0] % 128 == 0 and getattr(attn, "tp", None) is None)
        if not fusable:
            self._acquire(index, self._prefetch_target(prefetch_next))
            return layer.forward_prenorm(stream, pending, shape)
        unit = self.units[index]
        busy = set(self._resident.values())
        slot = next((s for s in range(len(self._full)) if s not in busy), None)
        if slot is None:
            raise RuntimeError("no free gather buffer: a unit was not released")
        weight = attn.qkv_proj
        n, k = weight._full_shape
        offset = self._offset_of(unit, weight)

        def produce(x2: torch.Tensor) -> torch.Tensor:
            _, out = self.fused_gather.gather_weight_gemm(
                x2, self.working[unit.base:unit.base + unit.shard], n, k, offset_elems=offset,
                out_flat=self._full[slot][:unit.padded])
            self._make_resident(index, slot)
            return out

        layer.norm1.weight.data = self._norm_cache[index]        # same values as the gathered copy that replaces it
        attn.qkv_override = lambda x: _GatherWeightLinearFn.apply(x, weight, produce)
        try:
            result = layer.forward_prenorm(stream, pending, shape)
        finally:
            attn.qkv_override = None
        target = self._prefetch_target(prefetch_next)
        if target is not None and self.prefetch:
            self._issue_gather(target)
        return result

    def _is_block(self, index: int) -> bool:
        return 1 <= index <= len(self.module.layers)

    def _prefetch_target(self, index: int | None) -> int | None:
        """Units that gather inside their own first GEMM are not prefetched."""
        if index is None or (self.fused_gather is not None and self._is_block(index)):
            return None
        return index

    # ------------------------------------------------------------------ compute
    def _embed(self, ids_flat: torch.Tensor, seq: int) -> torch.Tensor:
        m = self.module
        stream = m.token_embeddings(ids_flat)
        if m.position_embeddings is not None:
            positions = torch.arange(seq, device=ids_flat.device).repeat(ids_flat.numel() // seq)
            stream = stream + m.position_embeddings(positions)
        return stream

    def _head_weight(self) -> torch.Tensor:
        m = self.module
        return m.token_embeddings.weight if m.tie_embeddings else m.lm_head.weight

    def _borrow_embedding(self) -> None:
        """Tied head: gather the embedding unit into a private buffer and point the weight at it."""
        unit0 = self.units[0]
        borrowed = torch.empty(unit0.padded, dtype=self.dtype, device=self.device)
        dist.all_gather_into_tensor(borrowed, self.working[unit0.base:unit0.base + unit0.shard], group=self.group)
        emb = self.module.token_embeddings.weight
        off = unit0.offsets[unit0.params.index(emb)]
        emb.data = borrowed[off:off + emb._full_shape.numel()].view(emb._full_shape)

    def _return_embedding(self) -> None:
        emb = self.module.token_embeddings.weight
        emb.data = torch.empty(0, dtype=self.dtype, device=self.device)

    def _forward_only(self, token_ids, targets) -> torch.Tensor:
        m, n = self.module, len(self.units)
        B, T = token_ids.shape
        self._acquire(0, self._prefetch_target(1))
        stream = self._embed(token_ids.reshape(-1), T)
        self._release(0)
        pending = None
        for i, layer in enumerate(m.layers, start=1):
            stream, pending = self._run_block(i, layer, stream, pending, (B, T), i + 1 if i + 1 < n else None)
            self._release(i)
        self._acquire(n - 1)
        if m.tie_embeddings:
            self._borrow_embedding()
        hidden = m.final_norm.add_and_norm(stream, pending)[1]
        if targets is None:
            out = ops.linear(hidden, self._head_weight()).reshape(B, T, -1)
        else:
            out = ops.linear_cross_entropy(hidden, self._head_weight(), targets.reshape(-1))
        self._release(n - 1)
        if m.tie_embeddings:
            self._return_embedding()
        return out

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        with torch.no_grad():
            return self._forward_only(token_ids, None)

    def loss(self, token_ids: torch.Tensor, targets: torch.Tensor, loss_scale: float = 1.0) -> torch.Tensor:
        """Mean loss of this rank's batch. With autograd enabled the backward pass has already run when
        this returns (gradient shards hold ``loss_scale / world`` times this rank's gradient, summed over
        ranks); the returned tensor carries no graph and ``.backward()`` on it is a no-op."""
        if not torch.is_grad_enabled():
            return self._forward_only(token_ids, targets)
        m, n = self.module, len(self.units)
        B, T = token_ids.shape
        scale = loss_scale / self.world
        tied = m.tie_embeddings
        ids_flat = token_ids.reshape(-1)
        # ---- forward without autograd, remembering each unit's input
        with torch.no_grad():
            self._acquire(0, self._prefetch_target(1))
            stream = self._embed(ids_flat, T)
            self._release(0)
            pending = None
            saved = []
            for i, layer in enumerate(m.layers, start=1):
                saved.append((stream, pending))
                stream, pending = self._run_block(i, layer, stream, pending, (B, T), i + 1 if i + 1 < n else None)
                self._release(i)
        # ---- head: forward + backward with autograd
        head = n - 1
        self._acquire(head, self._prefetch_target(head - 1 if head - 1 >= 1 else None))
        self._attach_grad_views(self.units[head])
        tied_grad = None
        if tied:
            # the head borrows the embedding matrix: gather it into a private buffer for this stage
            self._borrow_embedding()
            emb = m.token_embeddings.weight
            tied_grad = torch.zeros(emb._full_shape, dtype=torch.float32, device=self.device)
            emb.main_grad = tied_grad
        stream = stream.detach().requires_grad_(True)
        pending_in = pending.detach().requires_grad_(True) if pending is not None else None
        with torch.enable_grad():
            hidden = m.final_norm.add_and_norm(stream, pending_in)[1]
            loss = ops.linear_cross_entropy(hidden, self._head_weight(), targets.reshape(-1), scale)
        loss.backward()
        grad_stream = stream.grad
        grad_pending = pending_in.grad if pending_in is not None else None
        if tied:
            emb = m.token_embeddings.weight
            if emb.grad is not None:
                tied_grad.add_(emb.grad.float())
                emb.grad = None
            emb.main_grad = None
            emb.data = torch.empty(0, dtype=self.dtype, device=self.device)
        self._reduce_unit_grads(head)
        self._release(head)
        loss_value = loss.detach()
        # ---- blocks in reverse: recompute with autograd, back-propagate, reduce-scatter
        for i in range(len(m.layers), 0, -1):
            layer = m.layers[i - 1]
            self._attach_grad_views(self.units[i])
            s_in, p_in = saved[i - 1]
            s_in = s_in.detach().requires_grad_(True)
            p_req = p_in.detach().requires_grad_(True) if p_in is not None else None
            with torch.enable_grad():
                s_out, p_out = self._run_block(i, layer, s_in, p_req, (B, T), i - 1 if i - 1 >= 1 else 0)
                outs, grads = [s_out, p_out], [grad_stream, grad_pending]
                aux = getattr(layer.feed_forward, "last_aux_loss", None)
                if aux is not None and aux.requires_grad:
                    outs.append(aux)
                    grads.append(torch.tensor(scale, dtype=aux.dtype, device=aux.device))
                    loss_value = loss_value + aux.detach()
            torch.autograd.backward(outs, grads)
            grad_stream, grad_pending = s_in.grad, (p_req.grad if p_req is not None else None)
            saved[i - 1] = None
            self._reduce_unit_grads(i)
            self._release(i)
        # ---- embeddings
        self._acquire(0)
        self._attach_grad_views(self.units[0])
        with torch.enable_grad():
            stream = self._embed(ids_flat, T)
        total = grad_stream if grad_pending is None else grad_stream + grad_pending
        stream.backward(total)
        if tied_grad is not None:
            m.token_embeddings.weight.main_grad.add_(tied_grad)
        self._reduce_unit_grads(0)
        self._release(0)
        # work queued on the current stream after this call sees complete gradient shards: the reductions that ran
        # beside the backward pass are joined here (a stream dependency, no host wait)
        self.join_reductions()
        # a leaf that accepts .backward(): the gradients above are already in place
        return loss_value.detach().clone().requires_grad_(True)

    # ------------------------------------------------------------------ checkpoint views
    @property
    def context_length(self) -> int:
        return self.module.context_length

    def export_named(self, sharded: torch.Tensor, local: torch.Tensor | None = None) -> dict[str, torch.Tensor]:
        """Gather a rank-sharded flat buffer and present it under the model's checkpoint key names (CPU, fp32)."""
        out: dict[str, torch.Tensor] = {}
        saved_local = []
        if local is not None:
            for (_, p), off in zip(self.local_named, self.local_offsets):
                saved_local.append(p.data)
                p.data = local[off:off + p.numel()].view(p.shape)
        try:
            for unit in self.units:
                full = torch.empty(unit.padded, dtype=sharded.dtype, device=self.device)
                dist.all_gather_into_tensor(full, sharded[unit.base:unit.base + unit.shard].contiguous(), group=self.group)
                for p, off in zip(unit.params, unit.offsets):
                    p.data = full[off:off + p._full_shape.numel()].view(p._full_shape)
                for prefix, mod in unit.modules:
                    for key, value in mod.state_dict(prefix=prefix).items():
                        out[key] = value.detach().float().cpu().clone()
                for p in unit.params:
                    p.data = torch.empty(0, dtype=self.dtype, device=self.device)
        finally:
            for (_, p), data in zip(self.local_named, saved_local):
                p.data = data
        order = list(self.module.state_dict_key_order()) if hasattr(self.module, "state_dict_key_order") else None
        if order:
            out = {k: out[k] for k in order if k in out} | {k: v for k, v in out.items() if k not in order}
        return out

    def import_named(self, named: dict[str, torch.Tensor], sharded: torch.Tensor, local: torch.Tensor | None = None) -> None:
        saved_local = []
        if local is not None:
            for (_, p), off in zip(self.local_named, self.local_offsets):
                saved_local.append(p.data)
                p.data = local[off:off + p.numel()].view(p.shape)
        try:
            for unit in self.units:
                full = torch.zeros(unit.padded, dtype=sharded.dtype, device=self.device)
                for p, off in zip(unit.params, unit.offsets):
                    p.data = full[off:off + p._full_shape.numel()].view(p._full_shape)
                for prefix, mod in unit.modules:
                    subset = {k[len(prefix):]: v.to(sharded.dtype) for k, v in named.items() if k.startswith(prefix)}
                    mod.load_state_dict(subset, strict=False)
                sharded[unit.base:unit.base + unit.shard].copy_(full[self.rank * unit.shard:(self.rank + 1) * unit.shard])
                for p in unit.params:
                    p.data = torch.empty(0, dtype=self.dtype, device=self.device)
        finally:
            for (_, p), data in zip(self.local_named, saved_local):
                p.data = data

    def state_dict(self, *args, **kwargs):          # model keys, un-sharded, un-prefixed
        merged = self.export_named(self.working, self.local_working)
        return {k: v.to(self.dtype) for k, v in merged.items()}

    def load_state_dict(self, state_dict, strict: bool = True):
        self.import_named(state_dict, self.working, self.local_working)
        if self.master is not self.working:
            self.master.copy_(self.working.float())
            if self.local_master is not None:
                self.local_master.copy_(self.local_working.float())
        self.refresh_norm_cache()
