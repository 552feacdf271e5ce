"""Continuous-batching scheduler.

Every engine step serves, in this order: running sequences that need a decode (or speculative
verify) step, then as many waiting requests as fit (``max_num_seqs`` sequences,
``max_batched_tokens`` new tokens, free KV blocks). Prompts longer than the remaining token budget
are prefilled in chunks. When a running sequence cannot get a block, the most recently admitted
running sequence is preempted: its blocks are released and it re-enters the waiting queue with its
generated tokens appended to its prompt (recompute on resume). The reference serves one prompt at a
time with no scheduler (``ajllm/workflows/lm_generate.py:56-81``).
"""

from __future__ import annotations

import itertools
from collections import deque
from dataclasses import dataclass, field
from enum import Enum

from ajllm_b200.engine.kv_cache import PagedKVCache


class SeqStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass
class SamplingParams:
    max_new_tokens: int = 100
    temperature: float = 0.8
    top_p: float | None = 0.95
    eos_token_id: int | None = None
    seed: int | None = None


@dataclass(eq=False)          # sequences are compared and hashed by identity (a field-wise == would walk the prompts)
class Sequence:
    request_id: int
    prompt: list[int]
    params: SamplingParams
    output: list[int] = field(default_factory=list)
    status: SeqStatus = SeqStatus.WAITING
    computed: int = 0                 # tokens whose K/V are in the cache
    preemptions: int = 0
    arrival: float = 0.0
    first_token_time: float | None = None
    finish_time: float | None = None
    finish_reason: str | None = None

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    def token_slice(self, start: int, stop: int) -> list[int]:
        """``tokens[start:stop]`` without joining prompt and output."""
        split = len(self.prompt)
        if stop <= split:
            return self.prompt[start:stop]
        if start >= split:
            return self.output[start - split:stop - split]
        return self.prompt[start:] + self.output[:stop - split]

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)

    @property
    def remaining_prefill(self) -> int:
        """Tokens (all but the one about to be predicted from) not yet in the cache."""
        return self.total_len - self.computed


@dataclass
class ScheduledSeq:
    seq: Sequence
    num_new_tokens: int       # tokens fed through the model this step
    is_prefill: bool
    samples: bool             # False for a non-final prefill chunk


class Scheduler:
    def __init__(self, cache: PagedKVCache, max_num_seqs: int = 256, max_batched_tokens: int = 8192,
                 context_length: int | None = None) -> None:
        self.cache = cache
        self.max_num_seqs = max_num_seqs
        self.max_batched_tokens = max_batched_tokens
        self.context_length = context_length
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []
        self._ids = itertools.count()
        self.num_preemptions = 0

    def add(self, prompt: list[int], params: SamplingParams, arrival: float = 0.0) -> Sequence:
        if not prompt:
            raise ValueError("a request needs at least one prompt token")
        if self.context_length is not None and len(prompt) >= self.context_length + 1:
            prompt = prompt[-self.context_length:]
        seq = Sequence(next(self._ids), list(prompt), params, arrival=arrival)
        self.waiting.append(seq)
        return seq

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ---------------------------------------------------------------- preemption
    def _preempt_youngest(self, protect: Sequence) -> bool:
        for victim in reversed(self.running):
            if victim is protect:
                continue
            self.running.remove(victim)
            self.cache.free(victim.request_id)
            victim.computed = 0
            victim.status = SeqStatus.WAITING
            victim.preemptions += 1
            self.num_preemptions += 1
            self.waiting.appendleft(victim)
            return True
        return False

    # ---------------------------------------------------------------- one step
    def schedule(self, decode_tokens: int = 1) -> list[ScheduledSeq]:
        """``decode_tokens`` is 1 for plain decoding and ``k + 1`` for a speculative verify step."""
        plan: list[ScheduledSeq] = []
        reserved: dict[int, int] = {}          # request id -> blocks promised to it in this plan
        promised = 0                           # their sum
        budget = self.max_batched_tokens

        def fits(seq: Sequence, new: int) -> bool:
            return self.cache.blocks_needed(seq.request_id, new) <= self.cache.allocator.free_blocks - promised

        # 1. running sequences (decode, or the next chunk of a long prefill)
        for seq in list(self.running):
            if seq.status is not SeqStatus.RUNNING:
                continue              # preempted while making room for an earlier sequence
            if seq.remaining_prefill > 1:
                new = min(seq.remaining_prefill, budget)
                is_prefill, samples = True, new == seq.remaining_prefill
            else:
                new, is_prefill, samples = decode_tokens, False, True
            if new <= 0 or new > budget:
                continue
            while not fits(seq, new):
                victim_count = len(self.running)
                if not self._preempt_youngest(seq):
                    break
                assert len(self.running) < victim_count
                for item in plan:
                    if item.seq.status is not SeqStatus.RUNNING:
                        budget += item.num_new_tokens
                        promised -= reserved.pop(item.seq.request_id, 0)
                plan = [item for item in plan if item.seq.status is SeqStatus.RUNNING]
            if not fits(seq, new):
                continue
            budget -= new
            reserved[seq.request_id] = self.cache.blocks_needed(seq.request_id, new)
            promised += reserved[seq.request_id]
            plan.append(ScheduledSeq(seq, new, is_prefill, samples))
        # 2. admit waiting requests
        while self.waiting and len(self.running) < self.max_num_seqs and budget > 0:
            seq = self.waiting[0]
            new = min(seq.remaining_prefill, budget)
            if not fits(seq, new):
                break
            self.waiting.popleft()
            seq.status = SeqStatus.RUNNING
            self.running.append(seq)
            budget -= new
            reserved[seq.request_id] = self.cache.blocks_needed(seq.request_id, new)
            promised += reserved[seq.request_id]
            plan.append(ScheduledSeq(seq, new, True, new == seq.remaining_prefill))
        if not plan and self.running and not self.waiting:
            raise RuntimeError("KV cache is too small to make progress on a single sequence")
        return plan

    def finish(self, seq: Sequence, reason: str, now: float = 0.0) -> None:
        seq.status = SeqStatus.FINISHED
        seq.finish_reason = reason
        seq.finish_time = now
        if seq in self.running:
            self.running.remove(seq)
        self.cache.free(seq.request_id)
