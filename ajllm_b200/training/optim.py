"""AdamW in the reference's update order, as a per-tensor optimizer and as a fused flat optimizer.

Update rule (``ajllm/training/optimizers.py:46-54``): ``m = b1 m + (1-b1) g``; ``v = b2 v + (1-b2) g^2``;
``p -= lr * sqrt(1-b2^t)/(1-b1^t) * m / (sqrt(v) + eps)``; then ``p *= 1 - lr * wd`` on the updated
parameter. Every parameter, norm gains included, is decayed, as in the reference's single group.

``FlatAdamW`` keeps all parameters of a model (or this rank's shards) in one contiguous buffer, with
fp32 master weights, fp32 moments and an fp32 gradient buffer that the backward kernels accumulate
into (``param.main_grad``). One kernel reduces the squared gradient norm, one kernel applies the clip
factor (read from device memory, no host sync) and the update, and writes the bf16 working copy.
Gradient clipping is by the true global norm over all ranks (the reference clips by a rank-local norm
under FSDP, ``ajllm/training/trainer.py:30-40``).
"""

from __future__ import annotations

import math
from typing import Any, Iterable

import torch
import torch.distributed as dist

from ajllm_b200.ops import native, reference


class AdamW(torch.optim.Optimizer):
    """Per-tensor AdamW with the reference's state layout (``step``, ``first_moment``, ``second_moment``)."""

    def __init__(self, parameters, learning_rate: float = 1e-3, betas: tuple[float, float] = (0.9, 0.999),
                 epsilon: float = 1e-8, weight_decay: float = 0.0) -> None:
        if learning_rate < 0:
            raise ValueError("learning_rate must be non-negative")
        if not (0 <= betas[0] < 1 and 0 <= betas[1] < 1):
            raise ValueError("Adam beta values must be in [0, 1)")
        super().__init__(parameters, {"lr": learning_rate, "betas": betas, "eps": epsilon,
                                      "weight_decay": weight_decay})

    @torch.no_grad()
    def step(self, closure=None):
        loss = closure() if closure is not None else None
        for group in self.param_groups:
            beta1, beta2 = group["betas"]
            for parameter in group["params"]:
                if parameter.grad is None:
                    continue
                state = self.state[parameter]
                if not state:
                    state["step"] = 0
                    state["first_moment"] = torch.zeros_like(parameter, dtype=torch.float32)
                    state["second_moment"] = torch.zeros_like(parameter, dtype=torch.float32)
                state["step"] += 1
                if parameter.dtype == torch.float32:
                    reference.adamw_update(parameter, parameter.grad, state["first_moment"], state["second_moment"],
                                           state["step"], group["lr"], beta1, beta2, group["eps"],
                                           group["weight_decay"])
                else:
                    master = state.setdefault("master", parameter.detach().float().clone())
                    reference.adamw_update(master, parameter.grad, state["first_moment"], state["second_moment"],
                                           state["step"], group["lr"], beta1, beta2, group["eps"],
                                           group["weight_decay"])
                    parameter.copy_(master)
        return loss


def _spec_groups(spec: dict, key: str) -> list:
    """Process groups of a parameter class: ``key`` (one group) and / or ``key + "s"`` (a list), ``None`` entries dropped."""
    groups = list(spec.get(key + "s") or [])
    if spec.get(key) is not None:
        groups.insert(0, spec[key])
    return [g for g in groups if g is not None]


def _group_sum_(value: torch.Tensor, group) -> torch.Tensor:
    if group is not None and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(value, op=dist.ReduceOp.SUM, group=group)
    return value


def clip_gradients(parameters: Iterable[torch.nn.Parameter], maximum_norm: float, epsilon: float = 1e-6) -> float:
    """Clip ``.grad`` tensors by their joint L2 norm and return that norm
    (``ajllm/training/trainer.py:30-40``)."""
    grads = [p.grad for p in parameters if p.grad is not None]
    if not grads:
        return 0.0
    total = torch.sqrt(sum(torch.sum(g.float().square()) for g in grads))
    norm = float(total)
    if norm > maximum_norm:
        factor = maximum_norm / (norm + epsilon)
        for g in grads:
            g.mul_(factor)
    return norm


# ------------------------------------------------------------------ flat primitives (CPU math / CUDA kernels)


_SCRATCH: dict = {}


def _sumsq_scratch(device: torch.device) -> torch.Tensor:
    """Per-device partial-sum buffer of the two-stage (fixed order, hence deterministic) reduction."""
    key = (device.type, device.index)
    if key not in _SCRATCH:
        _SCRATCH[key] = torch.empty(1024, dtype=torch.float32, device=device)
    return _SCRATCH[key]


def flat_sumsq(flat: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Sum of squares of an fp32 buffer as a 1-element fp32 tensor on the same device."""
    if flat.device.type == "cuda":
        out = torch.zeros(1, dtype=torch.float32, device=flat.device) if out is None else out.zero_()
        if flat.numel():
            native.call("ajb_sumsq_f32", flat.data_ptr(), flat.numel(), _sumsq_scratch(flat.device).data_ptr(),
                        out.data_ptr(), native.stream_ptr())
        return out
    value = flat.double().square().sum().float().reshape(1)
    if out is not None:
        out.copy_(value)
        return out
    return value


def flat_adamw(master: torch.Tensor, grad: torch.Tensor, m: torch.Tensor, v: torch.Tensor,
               working: torch.Tensor | None, step: int, lr: float, beta1: float, beta2: float, eps: float,
               weight_decay: float, sumsq: torch.Tensor | None, max_norm: float) -> None:
    """One AdamW step over flat fp32 buffers. The clip factor ``min(1, max_norm / (sqrt(sumsq)+1e-6))``
    is evaluated from the device scalar ``sumsq`` (``max_norm <= 0`` or ``sumsq is None`` disables it).
    ``working`` (bf16/fp16, may be ``None``) receives the updated parameters."""
    step_size = lr * math.sqrt(1 - beta2**step) / (1 - beta1**step)
    decay = 1.0 - lr * weight_decay
    if master.device.type == "cuda":
        native.call("ajb_adamw_flat", master.data_ptr(), grad.data_ptr(), m.data_ptr(), v.data_ptr(),
                    native.ptr(working), master.numel(), step_size, beta1, beta2, eps, decay,
                    native.ptr(sumsq), float(max_norm if sumsq is not None else 0.0), native.stream_ptr())
        return
    factor = 1.0
    if sumsq is not None and max_norm > 0:
        norm = float(sumsq.sqrt())
        if norm > max_norm:
            factor = max_norm / (norm + 1e-6)
    g = grad * factor
    m.mul_(beta1).add_(g, alpha=1 - beta1)
    v.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    master.addcdiv_(m, v.sqrt().add_(eps), value=-step_size)
    master.mul_(decay)
    if working is not None and working.data_ptr() != master.data_ptr():
        working.copy_(master)


class FlatAdamW:
    """Fused AdamW over one flat buffer holding every parameter of ``model`` that lives on this rank.

    ``reduce_plan`` lists ``(predicate, group)`` pairs: after backward, the gradient range of all
    parameters matching ``predicate`` is summed over ``group`` with a single collective (parameters are
    laid out so that each class is contiguous). ``norm_plan`` lists the groups over which each class's
    squared norm must be summed to obtain the global norm.
    """

    def __init__(self, model: torch.nn.Module, learning_rate: float = 1e-3, betas: tuple[float, float] = (0.9, 0.95),
                 epsilon: float = 1e-8, weight_decay: float = 0.0, classes: list[dict[str, Any]] | None = None) -> None:
        self.model = model
        self.defaults = {"lr": learning_rate, "betas": tuple(betas), "eps": epsilon, "weight_decay": weight_decay}
        self.param_groups = [dict(self.defaults)]
        self.step_count = 0
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        seen: set[int] = set()
        unique = []
        for name, p in named:
            if id(p) not in seen:
                seen.add(id(p))
                unique.append((name, p))
        # classes: [{"name", "match": fn(name, param)->bool, "reduce_group(s)", "norm_group(s)"}], first match wins;
        # the default single class needs no communication
        self.classes = classes or [{"name": "all", "match": lambda n, p: True, "reduce_group": None,
                                    "norm_group": None}]
        buckets: list[list[tuple[str, torch.nn.Parameter]]] = [[] for _ in self.classes]
        for name, p in unique:
            for index, spec in enumerate(self.classes):
                if spec["match"](name, p):
                    buckets[index].append((name, p))
                    break
            else:
                raise ValueError(f"parameter {name} matches no optimizer class")
        self.named_params = [item for bucket in buckets for item in bucket]
        device = self.named_params[0][1].device
        work_dtype = self.named_params[0][1].dtype
        align = 64  # elements; keeps every tensor 128-byte aligned in every buffer
        offsets, cursor, self.class_ranges = [], 0, []
        for bucket in buckets:
            begin = cursor
            for _, p in bucket:
                offsets.append(cursor)
                cursor += (p.numel() + align - 1) // align * align
            self.class_ranges.append((begin, cursor))
        self.total = cursor
        self.offsets = offsets
        self.working = torch.zeros(self.total, dtype=work_dtype, device=device)
        self.grad = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.m = torch.zeros(self.total, dtype=torch.float32, device=device)
        self.v = torch.zeros(self.total, dtype=torch.float32, device=device)
        for (name, p), off in zip(self.named_params, offsets):
            view = self.working[off:off + p.numel()].view(p.shape)
            view.copy_(p.data)
            p.data = view
            p.main_grad = self.grad[off:off + p.numel()].view(p.shape)
            p.main_grad_written = False
        self.master = self.working if work_dtype == torch.float32 else self.working.float()
        self._sumsq = torch.zeros(1, dtype=torch.float32, device=device)
        self._class_sumsq = torch.zeros(len(self.classes), dtype=torch.float32, device=device)

    # -------------------------------------------------------------- gradient plumbing
    def _join_side_streams(self) -> None:
        """Weight-gradient GEMMs may run on a side stream (``ops.functional.wgrad_accumulate``): everything that reads
        or clears the gradient buffer first makes the current stream wait for them."""
        if self.grad.is_cuda:
            from ajllm_b200.ops import functional
            functional.join_wgrad_stream()

    def zero_grad(self, set_to_none: bool = True) -> None:
        self._join_side_streams()
        self.grad.zero_()
        for _, p in self.named_params:
            p.grad = None
            p.main_grad_written = False

    @torch.no_grad()
    def collect_grads(self) -> None:
        """Fold autograd ``.grad`` tensors (ops that do not write ``main_grad`` themselves) into the flat buffer."""
        for _, p in self.named_params:
            if p.grad is not None:
                p.main_grad.add_(p.grad.to(torch.float32))
                p.grad = None

    @torch.no_grad()
    def reduce_grads(self) -> None:
        for spec, (begin, end) in zip(self.classes, self.class_ranges):
            for group in _spec_groups(spec, "reduce_group"):
                if end > begin and dist.get_world_size(group) > 1:
                    dist.all_reduce(self.grad[begin:end], op=dist.ReduceOp.SUM, group=group)

    @torch.no_grad()
    def global_sumsq(self) -> torch.Tensor:
        need_groups = any(_spec_groups(spec, "norm_group") for spec in self.classes)
        if not need_groups:
            return flat_sumsq(self.grad, self._sumsq)
        total = self._sumsq.zero_()
        for index, (spec, (begin, end)) in enumerate(zip(self.classes, self.class_ranges)):
            part = flat_sumsq(self.grad[begin:end]) if end > begin else torch.zeros_like(total)
            for group in _spec_groups(spec, "norm_group"):
                _group_sum_(part, group)
            total += part
        return total

    # -------------------------------------------------------------- update
    @torch.no_grad()
    def step(self, max_norm: float = 0.0) -> torch.Tensor:
        """Reduce, clip by global norm, update. Returns the (pre-clip) gradient norm as a device scalar."""
        self._join_side_streams()
        self.collect_grads()
        self.reduce_grads()
        sumsq = self.global_sumsq()
        self.step_count += 1
        group = self.param_groups[0]
        beta1, beta2 = group["betas"]
        flat_adamw(self.master, self.grad, self.m, self.v,
                   None if self.master is self.working else self.working, self.step_count, group["lr"],
                   beta1, beta2, group["eps"], group["weight_decay"], sumsq, max_norm)
        return sumsq.sqrt()

    # -------------------------------------------------------------- reference-format state
    def _export_through_model(self, flat: torch.Tensor) -> dict[str, torch.Tensor]:
        """Present a flat fp32 buffer under the model's checkpoint key names."""
        saved = []
        for (_, p), off in zip(self.named_params, self.offsets):
            saved.append(p.data)
            p.data = flat[off:off + p.numel()].view(p.shape)
        try:
            return {k: v.detach().float().cpu().clone() for k, v in self.model.state_dict().items()}
        finally:
            for (_, p), data in zip(self.named_params, saved):
                p.data = data

    def _import_through_model(self, named: dict[str, torch.Tensor], flat: torch.Tensor) -> None:
        saved = []
        for (_, p), off in zip(self.named_params, self.offsets):
            saved.append(p.data)
            p.data = flat[off:off + p.numel()].view(p.shape)
        try:
            self.model.load_state_dict({k: v.to(flat.dtype) for k, v in named.items()})
        finally:
            for (_, p), data in zip(self.named_params, saved):
                p.data = data

    def state_dict(self) -> dict[str, Any]:
        """``torch.optim``-shaped state in checkpoint-key order: ``state[i] = {step, first_moment,
        second_moment}`` for the i-th tensor of ``model.state_dict()``, plus ``param_names``."""
        first = self._export_through_model(self.m)
        second = self._export_through_model(self.v)
        names = list(first)
        state = {i: {"step": self.step_count, "first_moment": first[n], "second_moment": second[n]}
                 for i, n in enumerate(names)} if self.step_count else {}
        group = dict(self.param_groups[0])
        group["params"] = list(range(len(names)))
        out = {"state": state, "param_groups": [group], "param_names": names}
        if self.master is not self.working:
            out["master_weights"] = self._export_through_model(self.master)
        return out

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        group = state_dict["param_groups"][0]
        for key in ("lr", "betas", "eps", "weight_decay"):
            if key in group:
                self.param_groups[0][key] = tuple(group[key]) if key == "betas" else group[key]
        state = state_dict.get("state") or {}
        names = state_dict.get("param_names") or list(self.model.state_dict().keys())
        if state:
            entries = [state[k] for k in sorted(state, key=int)]
            self.step_count = int(entries[0]["step"])
            self._import_through_model({n: e["first_moment"] for n, e in zip(names, entries)}, self.m)
            self._import_through_model({n: e["second_moment"] for n, e in zip(names, entries)}, self.v)
        if self.master is not self.working:
            masters = state_dict.get("master_weights")
            if masters is not None:
                self._import_through_model(masters, self.master)
            else:
                self.master.copy_(self.working.float())
