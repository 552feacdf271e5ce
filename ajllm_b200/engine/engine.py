"""Request-level serving loop: scheduler + model runner + sampler (+ draft model).

``LLMEngine.generate`` is the batch entry point used by the workflows and the serving benchmark;
``add_request`` / ``step`` expose the same loop incrementally. Output token throughput is measured as
generated tokens divided by the time spent inside ``step`` calls.
"""

from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from ajllm_b200.engine.kv_cache import PagedKVCache
from ajllm_b200.engine.model_runner import ModelRunner, RunItem
from ajllm_b200.engine.scheduler import SamplingParams, ScheduledSeq, Scheduler, Sequence
from ajllm_b200.engine.spec_decode import verify_greedy, verify_rejection
from ajllm_b200.generation.sampling import sample_next_token, sampling_probabilities


@dataclass
class EngineStats:
    steps: int = 0
    prompt_tokens: int = 0
    output_tokens: int = 0
    draft_proposed: int = 0
    draft_accepted: int = 0
    busy_seconds: float = 0.0
    preemptions: int = 0

    @property
    def output_tokens_per_second(self) -> float:
        return self.output_tokens / self.busy_seconds if self.busy_seconds > 0 else 0.0

    @property
    def acceptance_rate(self) -> float:
        return self.draft_accepted / self.draft_proposed if self.draft_proposed else 0.0


@dataclass
class RequestOutput:
    request_id: int
    prompt: list[int]
    output: list[int]
    finish_reason: str | None
    preemptions: int = 0
    latency_seconds: float | None = None
    extras: dict = field(default_factory=dict)


def default_num_blocks(model, block_size: int, max_num_seqs: int) -> int:
    per_seq = (model.context_length + block_size - 1) // block_size
    return max(per_seq + 1, min(max_num_seqs * per_seq, 1 << 16))


def _cache_head_dim(head_dim: int, dtype, device) -> int:
    """Width of a cached head: on a GPU the attention kernels' head size (other sizes are stored zero-padded)."""
    if device.type == "cuda" and dtype == torch.bfloat16:
        from ajllm_b200.ops.functional import kernel_head_dim
        return kernel_head_dim(head_dim)
    return head_dim


class LLMEngine:
    def __init__(self, model, block_size: int = 16, num_blocks: int | None = None, max_num_seqs: int = 256,
                 max_batched_tokens: int = 8192, quantization: str | None = None, draft_model=None,
                 num_speculative_tokens: int = 4, seed: int = 0) -> None:
        model.eval()
        self.model = model
        device = next(model.parameters()).device
        dtype = next(model.parameters()).dtype
        attn = model.layers[0].attention
        num_blocks = num_blocks or default_num_blocks(model, block_size, max_num_seqs)
        self.cache = PagedKVCache(model.num_layers, num_blocks, block_size, attn.num_kv_heads,
                                  _cache_head_dim(attn.head_dim, dtype, device), dtype, device)
        self.runner = ModelRunner(model, self.cache, quantization)
        self.scheduler = Scheduler(self.cache, max_num_seqs, max_batched_tokens, model.context_length)
        self.k = num_speculative_tokens if draft_model is not None else 0
        self.draft_runner = None
        if draft_model is not None:
            draft_model.eval()
            dattn = draft_model.layers[0].attention
            self.draft_cache = PagedKVCache(draft_model.num_layers, num_blocks, block_size, dattn.num_kv_heads,
                                            _cache_head_dim(dattn.head_dim, dtype, device), dtype, device)
            self.draft_runner = ModelRunner(draft_model, self.draft_cache, None)
        self.stats = EngineStats()
        self.seed = seed
        self._generators: dict[int, torch.Generator] = {}
        self._draws: dict[int, int] = {}
        self._sampling_state = None          # (key, temps, top_ps, seeds, counters) of the previous sampling call
        self._finished: list[Sequence] = []

    # ---------------------------------------------------------------- requests
    def add_request(self, prompt: list[int], params: SamplingParams | None = None) -> int:
        params = params or SamplingParams()
        seq = self.scheduler.add(prompt, params, arrival=time.perf_counter())
        gen = torch.Generator(device="cpu")
        gen.manual_seed(params.seed if params.seed is not None else self.seed * 1_000_003 + seq.request_id)
        self._generators[seq.request_id] = gen
        return seq.request_id

    def has_unfinished(self) -> bool:
        return self.scheduler.has_work()

    # ---------------------------------------------------------------- helpers
    def _sample(self, seq: Sequence, logits_row: torch.Tensor) -> int:
        p = seq.params
        token = sample_next_token(logits_row[None].cpu(), p.temperature, p.top_p, self._generators[seq.request_id])
        return int(token[0, 0])

    def _sample_rows(self, seqs: list[Sequence], logits: torch.Tensor) -> list[int]:
        """One token per row of ``logits``. On the CPU every request draws from its own generator (results
        do not depend on batch composition); on a GPU the whole batch is sampled on the device and read
        back once, greedy rows by argmax and the rest from one device generator."""
        if not seqs:
            return []
        if logits.device.type != "cuda":
            return [self._sample(seq, logits[i]) for i, seq in enumerate(seqs)]
        from ajllm_b200.ops import serving
        temps, top_ps, seeds, counters = self._device_sampling_state(seqs, logits.device, draws=1)
        return serving.sample_rows(logits.float(), temps, top_ps, seeds, counters).tolist()

    def _device_sampling_state(self, seqs: list[Sequence], device, draws: int):
        """Per-row temperature / top-p / (seed, counter) tensors; advances each request's draw counter. While the batch
        keeps its composition (the usual case between two arrivals or departures) the tensors of the previous step are
        reused and the counters advance on the device."""
        key = (draws, tuple(s.request_id for s in seqs))
        cached = self._sampling_state
        if cached is not None and cached[0] == key and cached[1].device == device:
            _, temps, top_ps, seeds, counters = cached
            counters.add_(draws)
            for s in seqs:
                self._draws[s.request_id] += draws
            return temps, top_ps, seeds, counters
        temps = torch.tensor([s.params.temperature for s in seqs], dtype=torch.float32, device=device)
        top_ps = torch.tensor([(s.params.top_p if s.params.top_p is not None else 1.0) for s in seqs],
                              dtype=torch.float32, device=device)
        seeds, counters = [], []
        for s in seqs:
            seed = s.params.seed if s.params.seed is not None else self.seed * 1_000_003 + s.request_id
            seeds.append(seed & 0x7FFFFFFFFFFFFFFF)
            counters.append(self._draws.get(s.request_id, 0))
            self._draws[s.request_id] = counters[-1] + draws
        state = (temps, top_ps, torch.tensor(seeds, dtype=torch.int64, device=device),
                 torch.tensor(counters, dtype=torch.int64, device=device))
        self._sampling_state = (key, *state)
        return state

    def _emit(self, seq: Sequence, token: int, now: float) -> bool:
        """Append a generated token; returns True when the sequence finished."""
        seq.output.append(token)
        self.stats.output_tokens += 1
        if seq.first_token_time is None:
            seq.first_token_time = now
        p = seq.params
        if p.eos_token_id is not None and token == p.eos_token_id:
            self._finish(seq, "eos", now)
            return True
        if len(seq.output) >= p.max_new_tokens:
            self._finish(seq, "length", now)
            return True
        if seq.total_len >= self.model.context_length + 1:
            self._finish(seq, "context", now)
            return True
        return False

    def _finish(self, seq: Sequence, reason: str, now: float) -> None:
        self.scheduler.finish(seq, reason, now)
        if self.draft_runner is not None:
            self.draft_cache.free(seq.request_id)
        self._generators.pop(seq.request_id, None)
        self._draws.pop(seq.request_id, None)
        self._finished.append(seq)

    def _sync_preempted(self) -> None:
        """Sequences the scheduler pushed back to the waiting queue lose their draft cache too."""
        if self.draft_runner is None:
            return
        for seq in self.scheduler.waiting:
            if seq.computed == 0 and self.draft_cache.length(seq.request_id) > 0:
                self.draft_cache.free(seq.request_id)

    # ---------------------------------------------------------------- one engine step
    @torch.no_grad()
    def step(self) -> list[RequestOutput]:
        tick = time.perf_counter()
        done_before = len(self._finished)
        plan = self.scheduler.schedule(decode_tokens=self.k + 1 if self.k else 1)
        self._sync_preempted()
        self.stats.preemptions = self.scheduler.num_preemptions
        prefill = [item for item in plan if item.is_prefill]
        decode = [item for item in plan if not item.is_prefill]
        if self.k and decode:
            # a verify pass scores positions total_len - 1 .. total_len + k - 1: sequences closer than k tokens
            # to the context limit take the plain one-token decode below for this step
            roomy = [item for item in decode if item.seq.total_len + self.k <= self.model.context_length]
            if roomy:
                self._speculative_decode(roomy)
            decode = [ScheduledSeq(item.seq, 1, False, True) for item in decode
                      if item.seq.total_len + self.k > self.model.context_length]
        items, owners = [], []
        for item in prefill + decode:
            seq = item.seq
            new = seq.token_slice(seq.computed, seq.computed + item.num_new_tokens)
            items.append(RunItem(seq.request_id, new, 1 if item.samples else 0))
            owners.append(item)
        if items:
            logits = self.runner.forward(items)
            if self.draft_runner is not None:
                # keep the draft cache in step with the target for prompt tokens
                self.draft_runner.forward([RunItem(i.seq_id, i.token_ids, 0) for i in items])
            now = time.perf_counter()
            sampling = [item.seq for item in owners if item.samples]
            tokens = self._sample_rows(sampling, logits)
            row = 0
            for item in owners:
                seq = item.seq
                seq.computed = self.cache.length(seq.request_id)
                if item.is_prefill:
                    self.stats.prompt_tokens += item.num_new_tokens
                if item.samples:
                    self._emit(seq, tokens[row], now)
                    row += 1
        self._check_kernels()
        self.stats.steps += 1
        self.stats.busy_seconds += time.perf_counter() - tick
        return [self._to_output(seq) for seq in self._finished[done_before:]]

    def _check_kernels(self) -> None:
        """With projections fused with their collective, a rank whose peer stopped answering returns early with
        incomplete sums: raise (``PeerTimeout``) instead of emitting tokens computed from them. The step has just read
        its tokens back, so the device is idle and the check costs one small copy."""
        tp = self.runner.tp
        if tp is not None and getattr(tp, "fused", None) is not None:
            from ajllm_b200.ops import native
            native.check_status()

    def _speculative_decode_gpu(self, decode: list[ScheduledSeq]) -> None:
        """Same step with logits kept on the device: the sampler kernel proposes, the verify kernel decides,
        and only the proposed tokens and the (accepted, next) pairs are read back."""
        from ajllm_b200.ops import serving

        k = self.k
        seqs = [item.seq for item in decode]
        device = next(self.model.parameters()).device
        drafts: list[list[int]] = [[] for _ in seqs]
        draft_logits = []
        for _ in range(k):
            items = []
            for seq, proposed in zip(seqs, drafts):
                have = self.draft_cache.length(seq.request_id)
                items.append(RunItem(seq.request_id, seq.token_slice(have, seq.total_len) + proposed[max(0, have - seq.total_len):], 1))
            logits = self.draft_runner.forward(items).float()
            temps, top_ps, seeds, counters = self._device_sampling_state(seqs, device, draws=1)
            top_ps = torch.ones_like(top_ps)          # the accept rule below compares plain softmax distributions
            tokens = serving.sample_rows(logits, temps, top_ps, seeds, counters)
            draft_logits.append(logits)
            for row, token in enumerate(tokens.tolist()):
                drafts[row].append(token)
        items = [RunItem(seq.request_id, seq.token_slice(seq.computed, seq.total_len) + proposed, k + 1) for seq, proposed in zip(seqs, drafts)]
        target = self.runner.forward(items).float().view(len(seqs), k + 1, -1)
        temps, _, seeds, counters = self._device_sampling_state(seqs, device, draws=2 * k + 1)
        verdict = serving.spec_verify(target, torch.stack(draft_logits, dim=1),
                                      torch.tensor(drafts, dtype=torch.int32, device=device), temps, seeds,
                                      counters).tolist()
        now = time.perf_counter()
        for row, seq in enumerate(seqs):
            accepted, next_token = verdict[row]
            self._apply_verdict(seq, drafts[row], accepted, next_token, now)

    def _apply_verdict(self, seq: Sequence, proposed: list[int], accepted: int, next_token: int, now: float) -> None:
        k = self.k
        self.stats.draft_proposed += k
        self.stats.draft_accepted += accepted
        base = seq.total_len          # tokens known before this step
        for token in proposed[:accepted] + [next_token]:
            if self._emit(seq, token, now):
                return
        # keep K/V of the old tokens and of the accepted drafts; the new last token is fed next step
        self.cache.truncate(seq.request_id, base + accepted)
        self.draft_cache.truncate(seq.request_id, min(self.draft_cache.length(seq.request_id), base + accepted))
        seq.computed = self.cache.length(seq.request_id)

    def _speculative_decode(self, decode: list[ScheduledSeq]) -> None:
        if next(self.model.parameters()).is_cuda and all(
                item.seq.params.temperature <= 0 or item.seq.params.top_p in (None, 1.0) for item in decode):
            return self._speculative_decode_gpu(decode)
        k = self.k
        seqs = [item.seq for item in decode]
        drafts: list[list[int]] = [[] for _ in seqs]
        draft_probs: list[list[torch.Tensor]] = [[] for _ in seqs]
        # --- draft proposes k tokens per sequence (k small forward passes of the draft model)
        for step in range(k):
            items = []
            for seq, proposed in zip(seqs, drafts):
                have = self.draft_cache.length(seq.request_id)
                known = seq.tokens + proposed
                items.append(RunItem(seq.request_id, known[have:], 1))
            logits = self.draft_runner.forward(items)
            for row, seq in enumerate(seqs):
                p = seq.params
                if p.temperature <= 0:
                    token = int(torch.argmax(logits[row]))
                    draft_probs[row].append(None)
                else:
                    probs = sampling_probabilities(logits[row:row + 1].cpu(), p.temperature, p.top_p)[0]
                    token = int(torch.multinomial(probs, 1, generator=self._generators[seq.request_id]))
                    draft_probs[row].append(probs)
                drafts[row].append(token)
        # --- target scores the last accepted token plus the k proposals in one pass
        items = [RunItem(seq.request_id, seq.token_slice(seq.computed, seq.total_len) + proposed, k + 1)
                 for seq, proposed in zip(seqs, drafts)]
        logits = self.runner.forward(items)
        now = time.perf_counter()
        for row, seq in enumerate(seqs):
            p = seq.params
            block = logits[row * (k + 1):(row + 1) * (k + 1)].cpu()
            proposal = torch.tensor(drafts[row])
            if p.temperature <= 0:
                accepted, next_token = verify_greedy(proposal, block)
            else:
                target = sampling_probabilities(block, p.temperature, p.top_p)
                accepted, next_token = verify_rejection(proposal, torch.stack(draft_probs[row]), target,
                                                        self._generators[seq.request_id])
            self._apply_verdict(seq, drafts[row], accepted, next_token, now)

    # ---------------------------------------------------------------- batch API
    def _to_output(self, seq: Sequence) -> RequestOutput:
        latency = (seq.finish_time - seq.arrival) if seq.finish_time is not None else None
        return RequestOutput(seq.request_id, list(seq.prompt[:len(seq.prompt)]), list(seq.output), seq.finish_reason,
                             seq.preemptions, latency)

    def warm_up(self) -> int:
        """Captures the CUDA graphs of all decoding (and, with a draft model, verification) steps up to the engine's
        concurrency limit before the first request arrives; a no-op where steps are not replayed from graphs (CPU,
        expert models, quantised weights under tensor parallelism). Returns the number of graphs held."""
        graphs = self.runner.capture_decode_graphs(self.scheduler.max_num_seqs, (1, self.k + 1) if self.k else (1,))
        if self.draft_runner is not None:
            graphs += self.draft_runner.capture_decode_graphs(self.scheduler.max_num_seqs, (1,))
        return graphs

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams] | None = None
                 ) -> list[RequestOutput]:
        if not isinstance(params, list):
            params = [params or SamplingParams()] * len(prompts)
        ids = [self.add_request(prompt, p) for prompt, p in zip(prompts, params)]
        finished: dict[int, RequestOutput] = {}
        while self.has_unfinished():
            for out in self.step():
                finished[out.request_id] = out
        return [finished[i] for i in ids]
