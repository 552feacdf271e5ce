"""Training loop that maintains a self-contained run directory.

Contract kept from the reference (``ajllm/training/trainer.py:43-210``): config keys and defaults
(``training.{batch_size=64, max_steps|total_tokens, gradient_clip=1.0, resume_from}``,
``optimizer.{max_lr=1e-3, min_lr|min_lr_ratio=0.1, beta1=0.9, beta2=0.95, epsilon=1e-8,
weight_decay=0.1}``, ``scheduler.warmup_steps=0``, ``logging.{log_interval=50, eval_interval=500,
eval_batches=20, checkpoint_interval=10000}``), ``metrics.jsonl`` events ``train`` / ``evaluation``,
``checkpoints/step_%08d.pt`` + ``final.pt``, ``summary.json`` keys.

Differences, all deliberate: ``latest.pt`` is refreshed at every checkpoint and ``best.pt`` whenever
the validation loss improves (the reference documents both and writes neither); gradients may be
accumulated over ``training.gradient_accumulation_steps`` micro-batches; the clip norm is global
across ranks; the loss is read back only when a record is logged (no per-step host sync); batches are
staged through pinned memory by a worker thread; each data-parallel rank draws different windows
(``training.identical_rank_batches: true`` restores the reference's behaviour); the data RNG state is
checkpointed; ``tokens_per_second`` excludes evaluation/checkpoint time and a device-timed
``tokens_per_second_device_max`` (max over ranks) is logged next to it.
"""

from __future__ import annotations

import json
import math
import time
from pathlib import Path
from typing import Any

import numpy as np
import torch
import torch.distributed as dist

from ajllm_b200.training.checkpoint import load_checkpoint, save_checkpoint
from ajllm_b200.training.data import BatchStager
from ajllm_b200.training.logger import RunLogger
from ajllm_b200.training.optim import FlatAdamW
from ajllm_b200.training.schedulers import warmup_cosine_learning_rate
from ajllm_b200.utils.timing import max_over_ranks


def is_main_process() -> bool:
    return not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0


def _mean_over_group(value: torch.Tensor, group=None) -> torch.Tensor:
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        value = value.clone()
        dist.all_reduce(value, op=dist.ReduceOp.SUM, group=group)
        value /= dist.get_world_size(group)
    return value


def optimizer_step(model, optimizer, next_batch, accumulation: int, gradient_clip: float):
    """One optimisation step: ``accumulation`` micro-batches of forward + backward, then the clipped
    AdamW update. ``next_batch()`` yields device ``(inputs, targets)``. Returns ``(loss, grad_norm)`` as
    device scalars (the loss is the mean over the micro-batches); nothing is read back to the host."""
    optimizer.zero_grad(set_to_none=True)
    total = None
    together = int(getattr(model, "interleave", 1))
    if together > 1 and accumulation % together == 0:
        # several micro-batches in flight: their kernels alternate block by block on streams of their own
        for _ in range(accumulation // together):
            batches = [next_batch() for _ in range(together)]
            losses = model.loss_interleaved(batches, 1.0 / accumulation)
            torch.autograd.backward(losses)
            model.join_streams()
            for loss in losses:
                piece = loss.detach().float() / accumulation
                total = piece if total is None else total + piece
        return total, optimizer.step(gradient_clip)
    for _ in range(accumulation):
        inputs, targets = next_batch()
        loss = model.loss(inputs, targets, 1.0 / accumulation)
        loss.backward()
        piece = loss.detach().float() / accumulation
        total = piece if total is None else total + piece
    join = getattr(model, "join_streams", None)
    if join is not None and total is not None and total.is_cuda:
        join()              # weight gradients issued on the side stream are complete before the optimizer reads them
    return total, optimizer.step(gradient_clip)


class Trainer:
    def __init__(self, model: torch.nn.Module, train_dataset, validation_dataset, run_directory: str | Path,
                 config: dict[str, Any], device: torch.device, seed: int, optimizer=None,
                 data_rank: int = 0, data_world: int = 1, loss_reduce_group=None) -> None:
        self.model = model
        self.train_dataset, self.validation_dataset = train_dataset, validation_dataset
        self.run_directory = Path(run_directory)
        self.config, self.device, self.seed = config, device, seed
        training = config.get("training", {})
        identical = bool(training.get("identical_rank_batches", False))
        self.data_rank, self.data_world = data_rank, data_world
        # ranks of one tensor-parallel group share data_rank and therefore draw the same windows
        self.generator = np.random.default_rng(seed if identical else [seed, data_rank])
        self.logger = RunLogger(self.run_directory) if is_main_process() else None
        self.loss_reduce_group = loss_reduce_group

        opt = config.get("optimizer", {})
        self.maximum_learning_rate = float(opt.get("max_lr", 1e-3))
        self.minimum_learning_rate = float(
            opt.get("min_lr", self.maximum_learning_rate * float(opt.get("min_lr_ratio", 0.1))))
        self.optimizer = optimizer if optimizer is not None else FlatAdamW(
            model,
            learning_rate=self.maximum_learning_rate,
            betas=(float(opt.get("beta1", 0.9)), float(opt.get("beta2", 0.95))),
            epsilon=float(opt.get("epsilon", 1e-8)),
            weight_decay=float(opt.get("weight_decay", 0.1)),
        )

    # ------------------------------------------------------------------ helpers
    @property
    def base_model(self):
        return getattr(self.model, "module", self.model)

    def _loss(self, inputs, targets, loss_scale: float = 1.0) -> torch.Tensor:
        if hasattr(self.model, "loss"):
            return self.model.loss(inputs, targets, loss_scale)
        from ajllm_b200.training.losses import cross_entropy
        return cross_entropy(self.model(inputs), targets) * loss_scale

    def _global_loss(self, local: torch.Tensor) -> float:
        """Device scalar -> host float of the global mean loss (ranks hold shares or replicas)."""
        value = local.detach().float().reshape(1)
        for axis in (getattr(self.base_model, "tp", None), getattr(self.base_model, "cp", None)):
            if axis is not None and axis.size > 1:
                value = value.clone()
                dist.all_reduce(value, op=dist.ReduceOp.SUM, group=axis.group)   # shares add up to the mean
        if self.loss_reduce_group is not None:
            if float(getattr(self.base_model, "data_parallel_share", 1.0)) != 1.0:
                value = value.clone()           # replicas report local_mean / dp: the shares add up to the mean
                dist.all_reduce(value, op=dist.ReduceOp.SUM, group=self.loss_reduce_group)
            else:
                value = _mean_over_group(value, self.loss_reduce_group)
        return float(value.item())

    @torch.no_grad()
    def evaluate(self, batches: int, batch_size: int, context_length: int) -> dict[str, float]:
        self.model.eval()
        results: dict[str, float] = {}
        for name, dataset in (("train", self.train_dataset), ("validation", self.validation_dataset)):
            if dataset is None:
                continue
            total = 0.0
            for _ in range(batches):
                inputs, targets = dataset.batch(batch_size, context_length, self.device, self.generator)
                total += self._global_loss(self._loss(inputs, targets))
            results[f"{name}_loss"] = total / batches
            results[f"{name}_perplexity"] = math.exp(min(results[f"{name}_loss"], 50.0))
        self.model.train()
        return results

    def _check_kernels(self) -> None:
        """Raise :class:`ajllm_b200.ops.native.PeerTimeout` when a kernel of this rank gave up a bounded wait
        (its outputs, e.g. reduced gradients, are then incomplete). Synchronises the device."""
        if self.device.type == "cuda":
            from ajllm_b200.ops import native
            native.check_status()

    def _save(self, path: Path, step: int, metadata: dict[str, Any], best_validation_loss: float,
              aliases: tuple[str, ...] = ()) -> Path:
        """Checkpoint entered by every rank (state gathering is collective); refused after a kernel timeout so
        that weights updated from incomplete gradients never reach the disk."""
        self._check_kernels()
        return save_checkpoint(path, self.model, self.optimizer, step, metadata,
                               self._extra_state(best_validation_loss), aliases=aliases)

    def _agreed(self, flag: bool) -> bool:
        """Rank 0's view of a file-system fact, so that every rank takes the same branch into a collective."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            return flag
        box = [flag]
        dist.broadcast_object_list(box, src=0)
        return bool(box[0])

    def _extra_state(self, best_validation_loss: float) -> dict[str, Any]:
        return {"data_rng_state": self.generator.bit_generator.state, "best_validation_loss": best_validation_loss}

    # ------------------------------------------------------------------ main loop
    def train(self, checkpoint_metadata: dict[str, Any]) -> dict[str, Any]:
        training = self.config.get("training", {})
        logging = self.config.get("logging", {})
        batch_size = int(training.get("batch_size", 64))
        accumulation = max(1, int(training.get("gradient_accumulation_steps", 1)))
        context_length = int(self.base_model.context_length)
        tokens_per_step = batch_size * context_length * accumulation * self.data_world
        if "max_steps" in training:
            max_steps = int(training["max_steps"])
        elif "total_tokens" in training:
            max_steps = max(1, int(training["total_tokens"]) // tokens_per_step)
        else:
            raise ValueError("training.max_steps or training.total_tokens is required")
        warmup_steps = int(self.config.get("scheduler", {}).get("warmup_steps", 0))
        gradient_clip = float(training.get("gradient_clip", 1.0))
        log_interval = int(logging.get("log_interval", 50))
        eval_interval = int(logging.get("eval_interval", 500))
        eval_batches = int(logging.get("eval_batches", 20))
        checkpoint_interval = int(logging.get("checkpoint_interval", 10000))
        checkpoint_directory = self.run_directory / "checkpoints"
        if is_main_process():
            checkpoint_directory.mkdir(parents=True, exist_ok=True)

        start_step, best_validation_loss = 0, float("inf")
        resume_from = training.get("resume_from")
        if resume_from:
            checkpoint = load_checkpoint(resume_from, self.model, self.optimizer, self.device)
            start_step = int(checkpoint["step"])
            if "data_rng_state" in checkpoint and self.data_rank == 0 and self.data_world == 1:
                self.generator.bit_generator.state = checkpoint["data_rng_state"]
            best_validation_loss = float(checkpoint.get("best_validation_loss", best_validation_loss))

        use_cuda = self.device.type == "cuda"
        stager = BatchStager(self.train_dataset, batch_size, context_length, self.device, self.generator)
        self.model.train()
        train_seconds = 0.0           # host time spent in optimisation steps only
        device_ms = 0.0               # CUDA-event time of the same steps
        steps_timed = 0
        pending_events: list[tuple[Any, Any]] = []
        training_started = time.perf_counter()
        loss_value = torch.zeros((), device=self.device)
        try:
            for step in range(start_step, max_steps):
                learning_rate = warmup_cosine_learning_rate(
                    step, self.maximum_learning_rate, self.minimum_learning_rate, warmup_steps, max_steps)
                for group in self.optimizer.param_groups:
                    group["lr"] = learning_rate
                tick = time.perf_counter()
                if use_cuda:
                    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    begin.record()
                loss_value, gradient_norm = optimizer_step(self.model, self.optimizer, stager.next, accumulation,
                                                           gradient_clip)
                if use_cuda:
                    end.record()
                    pending_events.append((begin, end))
                train_seconds += time.perf_counter() - tick
                steps_timed += 1
                completed = step + 1

                if completed % log_interval == 0 or completed == 1:
                    if use_cuda:
                        self._check_kernels()         # synchronises; a timed-out wait stops the run here
                        device_ms += sum(b.elapsed_time(e) for b, e in pending_events)
                        pending_events.clear()
                    loss_float = self._global_loss(loss_value)
                    device_rate = None
                    if use_cuda and device_ms > 0:
                        device_rate = steps_timed * tokens_per_step / (max_over_ranks(device_ms, self.device) / 1e3)
                    if self.logger is not None:
                        record = {
                            "loss": loss_float,
                            "learning_rate": learning_rate,
                            "gradient_norm": float(gradient_norm),
                            "tokens_per_second": steps_timed * tokens_per_step / max(train_seconds, 1e-9),
                        }
                        if device_rate is not None:
                            record["tokens_per_second_device_max"] = device_rate
                        self.logger.log(completed, "train", record)

                if eval_interval > 0 and (completed % eval_interval == 0 or completed == max_steps):
                    evaluation = self.evaluate(eval_batches, batch_size, context_length)
                    if self.logger is not None:
                        self.logger.log(completed, "evaluation", evaluation)
                    validation_loss = evaluation.get("validation_loss")
                    if validation_loss is not None and validation_loss < best_validation_loss:
                        best_validation_loss = validation_loss
                        self._save(checkpoint_directory / "best.pt", completed, checkpoint_metadata,
                                   best_validation_loss)

                if checkpoint_interval > 0 and completed % checkpoint_interval == 0:
                    self._save(checkpoint_directory / f"step_{completed:08d}.pt", completed, checkpoint_metadata,
                               best_validation_loss, aliases=("latest.pt",))
        finally:
            stager.close()

        final_path = self._save(checkpoint_directory / "final.pt", max_steps, checkpoint_metadata,
                                best_validation_loss, aliases=("latest.pt",))
        final_evaluation = self.evaluate(eval_batches, batch_size, context_length)
        validation_loss = final_evaluation.get("validation_loss")
        best_path = checkpoint_directory / "best.pt"
        # every rank enters a save (state gathering is collective), so the decision uses only values all ranks share:
        # the evaluation result (already reduced over ranks) and rank 0's view of the file system
        best_missing = self._agreed(not best_path.exists())
        if validation_loss is not None and (validation_loss < best_validation_loss or best_missing):
            best_validation_loss = min(best_validation_loss, validation_loss)
            self._save(best_path, max_steps, checkpoint_metadata, best_validation_loss)
        elif validation_loss is None and best_missing:
            # no validation split: "best" resolves to the final weights
            self._save(best_path, max_steps, checkpoint_metadata, best_validation_loss)
        summary = {
            "status": "completed",
            "steps": max_steps,
            "tokens_seen": max_steps * tokens_per_step,
            "elapsed_seconds": time.perf_counter() - training_started,
            "best_validation_loss": None if math.isinf(best_validation_loss) else best_validation_loss,
            "checkpoint": str(final_path) if is_main_process() else None,
            **final_evaluation,
        }
        if is_main_process():
            with (self.run_directory / "summary.json").open("w", encoding="utf-8") as handle:
                json.dump(summary, handle, indent=2)
        return summary
