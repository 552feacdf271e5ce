"""Pipeline parallelism: contiguous groups of blocks on consecutive ranks, 1F1B micro-batch schedule.

The reference has no pipeline parallelism (its distributed module, ``ajllm/training/distributed.py``,
offers data, fully-sharded and tensor modes); this module covers the optional send/recv stage of the
parallel runtime. Stage 0 owns the embeddings, the last stage owns the final norm and the LM head, and
every stage owns ``num_layers / stages`` consecutive blocks. Activations and their gradients travel
between neighbours with ``torch.distributed`` point-to-point operations (NCCL on GPUs, gloo on CPUs),
batched per schedule slot (``batch_isend_irecv``) so that a stage that is sending forward while its
neighbour sends backward cannot block on it. With the one-forward-one-backward schedule a stage holds at
most ``stages - stage`` micro-batches of activations.

``PipelineParallel.loss`` runs the whole schedule, so, like the fully sharded wrapper, the backward pass
has happened when it returns, and the value it returns (the same on every stage) carries no graph.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ajllm_b200 import ops


def stage_bounds(num_layers: int, stages: int, stage: int) -> tuple[int, int]:
    """Blocks ``[lo, hi)`` of ``stage``: the first ``num_layers % stages`` stages take one more block."""
    base, extra = divmod(num_layers, stages)
    lo = stage * base + min(stage, extra)
    return lo, lo + base + (1 if stage < extra else 0)


class PipelineParallel(nn.Module):
    def __init__(self, model, group, num_microbatches: int) -> None:
        super().__init__()
        if model.norm_placement != "pre":
            raise ValueError("pipeline parallelism supports pre-norm models")
        if model.tie_embeddings:
            raise ValueError("tied embeddings would live on the first and the last stage; untie them for pipeline parallelism")
        self.group = group
        self.stage = dist.get_rank(group)
        self.stages = dist.get_world_size(group)
        if len(model.layers) < self.stages:
            raise ValueError("fewer blocks than pipeline stages")
        self.num_microbatches = int(num_microbatches)
        self.first, self.last = self.stage == 0, self.stage == self.stages - 1
        self.layer_lo, self.layer_hi = stage_bounds(len(model.layers), self.stages, self.stage)
        model.layers = nn.ModuleList(list(model.layers)[self.layer_lo:self.layer_hi])
        if not self.first:
            model.token_embeddings = None
            model.position_embeddings = None
        if not self.last:
            model.final_norm = None
            model.lm_head = None
        self.module = model
        first_param = next(model.parameters())
        self.device, self.dtype = first_param.device, first_param.dtype
        self.d_model = model.d_model
        self._prev = dist.get_global_rank(group, self.stage - 1) if not self.first else None
        self._next = dist.get_global_rank(group, self.stage + 1) if not self.last else None

    # ------------------------------------------------------------------ naming (checkpoints use whole-model keys)
    def global_name(self, local_name: str) -> str:
        if local_name.startswith("layers."):
            index, rest = local_name[len("layers."):].split(".", 1)
            return f"layers.{int(index) + self.layer_lo}.{rest}"
        return local_name

    def state_dict_global(self) -> dict[str, torch.Tensor]:
        """The whole model's state (every stage's tensors, whole-model keys) on every rank of the group."""
        mine = {self.global_name(k): v.detach().cpu() for k, v in self.module.state_dict().items()}
        parts: list[dict] = [None] * self.stages          # type: ignore[list-item]
        dist.all_gather_object(parts, mine, group=self.group)
        merged: dict[str, torch.Tensor] = {}
        for part in parts:
            merged.update(part)
        return merged

    def load_state_dict_global(self, state: dict[str, torch.Tensor]) -> None:
        own = {k: state[self.global_name(k)] for k in self.module.state_dict().keys()}
        self.module.load_state_dict(own)

    # ------------------------------------------------------------------ point-to-point slots
    def _exchange(self, send_next=None, send_prev=None, recv_prev: bool = False, recv_next: bool = False, shape=None):
        """One schedule slot: up to one tensor in each direction, posted together and waited for together."""
        ops_list, got_prev, got_next = [], None, None
        if recv_prev and self._prev is not None:
            got_prev = torch.empty(shape, dtype=self.dtype, device=self.device)
            ops_list.append(dist.P2POp(dist.irecv, got_prev, self._prev, group=self.group))
        if recv_next and self._next is not None:
            got_next = torch.empty(shape, dtype=self.dtype, device=self.device)
            ops_list.append(dist.P2POp(dist.irecv, got_next, self._next, group=self.group))
        if send_next is not None and self._next is not None:
            ops_list.append(dist.P2POp(dist.isend, send_next.contiguous(), self._next, group=self.group))
        if send_prev is not None and self._prev is not None:
            ops_list.append(dist.P2POp(dist.isend, send_prev.contiguous(), self._prev, group=self.group))
        if ops_list:
            for work in dist.batch_isend_irecv(ops_list):
                work.wait()
        return got_prev, got_next

    # ------------------------------------------------------------------ one micro-batch through this stage
    def _forward_micro(self, tokens: torch.Tensor, targets: torch.Tensor, x_in: torch.Tensor | None, scale: float):
        m = self.module
        B, T = tokens.shape
        if self.first:
            ids = tokens.reshape(-1)
            stream = m.token_embeddings(ids)
            if m.position_embeddings is not None:
                stream = stream + m.position_embeddings(torch.arange(T, device=tokens.device).repeat(B))
        else:
            stream = x_in
        pending = None
        for layer in m.layers:
            stream, pending = layer.forward_prenorm(stream, pending, (B, T))
        aux_terms = [layer.feed_forward.last_aux_loss for layer in m.layers
                     if getattr(layer.feed_forward, "last_aux_loss", None) is not None]
        aux = sum(aux_terms) * scale if aux_terms else None
        if self.last:
            hidden = m.final_norm.add_and_norm(stream, pending)[1]
            # the value is the unscaled mean of this micro-batch; `scale` multiplies its gradient only
            out = ops.linear_cross_entropy(hidden, m.head_weight, targets.reshape(-1), scale)
        else:
            out = stream if pending is None else stream + pending
        return out, aux

    def loss(self, token_ids: torch.Tensor, targets: torch.Tensor, loss_scale: float = 1.0) -> torch.Tensor:
        """Mean loss of the batch, identical on every stage. Gradients of this stage's parameters are in
        ``.grad`` / ``main_grad`` when this returns (scaled by ``loss_scale``)."""
        M = self.num_microbatches
        B, T = token_ids.shape
        if B % M:
            raise ValueError(f"batch of {B} sequences does not split into {M} micro-batches")
        per = B // M
        scale = loss_scale / M
        train = torch.is_grad_enabled()
        shape = (per * T, self.d_model)
        total = torch.zeros((), dtype=torch.float32, device=self.device)
        held: list[tuple] = []          # (x_in, out, aux) of micro-batches whose backward is still to come

        def forward(i: int, x_in):
            if x_in is not None and train:
                x_in.requires_grad_(True)
            sl = slice(i * per, (i + 1) * per)
            out, aux = self._forward_micro(token_ids[sl], targets[sl], x_in, scale)
            nonlocal total
            if self.last:
                total += out.detach().float() / M
            if aux is not None:
                total += aux.detach().float()
            held.append((x_in, out, aux))
            return out

        def backward(grad_out):
            x_in, out, aux = held.pop(0)
            outs, grads = [out], [grad_out]
            if self.last:
                grads = [None]
            if aux is not None:
                outs.append(aux)
                grads.append(None)
            torch.autograd.backward(outs, grads)
            return x_in.grad if x_in is not None else None

        if not train:
            for i in range(M):
                x_in, _ = self._exchange(recv_prev=True, shape=shape)
                out = forward(i, x_in)
                self._exchange(send_next=None if self.last else out)
                held.clear()
        else:
            warmup = min(self.stages - 1 - self.stage, M)
            steady = M - warmup
            for i in range(warmup):
                x_in, _ = self._exchange(recv_prev=True, shape=shape)
                out = forward(i, x_in)
                self._exchange(send_next=out.detach())
            x_in = self._exchange(recv_prev=True, shape=shape)[0] if steady > 0 else None
            for i in range(steady):
                out = forward(warmup + i, x_in)
                _, grad_out = self._exchange(send_next=None if self.last else out.detach(), recv_next=True, shape=shape)
                grad_in = backward(grad_out)
                if i + 1 < steady:
                    x_in, _ = self._exchange(send_prev=grad_in, recv_prev=True, shape=shape)
                else:
                    self._exchange(send_prev=grad_in)
            for _ in range(warmup):
                _, grad_out = self._exchange(recv_next=True, shape=shape)
                grad_in = backward(grad_out)
                self._exchange(send_prev=grad_in)
        # the last stage knows the language-model loss, earlier stages their auxiliary terms: sum over stages
        if self.stages > 1:
            dist.all_reduce(total, op=dist.ReduceOp.SUM, group=self.group)
        return total.detach().clone().requires_grad_(train)

    @property
    def context_length(self) -> int:
        return self.module.context_length

    def state_dict(self, *args, **kwargs):          # whole-model keys, every stage's tensors
        return self.state_dict_global()

    def load_state_dict(self, state_dict, strict: bool = True):
        self.load_state_dict_global(state_dict)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError("a pipeline stage has no whole-model forward; use loss() or gather the stages")


class PipelineOptimizer:
    """One stage's :class:`~ajllm_b200.training.optim.FlatAdamW` behind the optimizer surface the trainer uses, with
    whole-model state dicts: ``state_dict()`` gathers every stage's moments (and fp32 master weights) under
    whole-model parameter names in model order, ``load_state_dict()`` keeps this stage's part. A checkpoint written
    by a pipeline run therefore has the same layout as one written by a single process."""

    def __init__(self, pipe: PipelineParallel, **adamw_kwargs) -> None:
        from ajllm_b200.training.optim import FlatAdamW

        self.pipe = pipe
        self.inner = FlatAdamW(pipe.module, classes=pp_optimizer_classes(pipe.group), **adamw_kwargs)

    @property
    def param_groups(self):
        return self.inner.param_groups

    @property
    def step_count(self) -> int:
        return self.inner.step_count

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.inner.zero_grad(set_to_none)

    def step(self, max_norm: float = 0.0) -> torch.Tensor:
        return self.inner.step(max_norm)

    def state_dict(self) -> dict:
        local = self.inner.state_dict()
        names = [self.pipe.global_name(n) for n in local["param_names"]]
        mine = {"names": names,
                "entries": [local["state"][i] for i in range(len(names))] if local["state"] else [],
                "masters": {self.pipe.global_name(k): v.cpu() for k, v in local.get("master_weights", {}).items()}}
        for entry in mine["entries"]:
            entry["first_moment"], entry["second_moment"] = entry["first_moment"].cpu(), entry["second_moment"].cpu()
        parts: list[dict] = [None] * self.pipe.stages          # type: ignore[list-item]
        dist.all_gather_object(parts, mine, group=self.pipe.group)
        merged_names = [n for part in parts for n in part["names"]]
        merged_entries = [e for part in parts for e in part["entries"]]
        group = dict(local["param_groups"][0])
        group["params"] = list(range(len(merged_names)))
        out = {"state": dict(enumerate(merged_entries)), "param_groups": [group], "param_names": merged_names}
        masters = {k: v for part in parts for k, v in part["masters"].items()}
        if masters:
            out["master_weights"] = masters
        return out

    def load_state_dict(self, state_dict: dict) -> None:
        names = state_dict.get("param_names")
        if names is None:
            raise ValueError("an optimizer state without parameter names cannot be split over pipeline stages")
        own = {self.pipe.global_name(k): k for k in self.pipe.module.state_dict().keys()}
        picked = [(i, own[n]) for i, n in enumerate(names) if n in own]
        state = state_dict.get("state") or {}
        local = {"param_groups": [dict(state_dict["param_groups"][0], params=list(range(len(picked))))],
                 "param_names": [local_name for _, local_name in picked],
                 "state": {j: state[i] if i in state else state[str(i)] for j, (i, _) in enumerate(picked)} if state else {}}
        masters = state_dict.get("master_weights")
        if masters is not None:
            local["master_weights"] = {own[n]: v for n, v in masters.items() if n in own}
        self.inner.load_state_dict(local)


def pp_optimizer_classes(group) -> list[dict]:
    """Parameter classes for :class:`ajllm_b200.training.optim.FlatAdamW` on one pipeline stage: nothing to
    reduce (every parameter lives on exactly one stage) but the gradient norm is summed over the stages."""
    return [{"name": "stage", "match": lambda n, p: True, "reduce_group": None, "norm_group": group}]
