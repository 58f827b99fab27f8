"""The scheduler: every step, which sequences run and how many tokens each.

Continuous batching under two limits, `max_num_seqs` running sequences and
`max_num_batched_tokens` tokens per step (atomserve/scheduler.py:1-35, 88-135):

 1. Running sequences first, oldest first: one token for a decode, or the next portion of a
    prompt, as much as the budget leaves. When the cache has no pages for one, the most
    recently admitted sequence is preempted: everything it holds is given back and it returns
    to the front of the queue, to be recomputed from its tokens. If the sequence in need is
    itself the newest, it is the one preempted. Nothing is admitted in a step that preempted.
 2. Waiting sequences are admitted first come, first served, while budget, sequence limit,
    state slots and pages allow; the head of the queue is never skipped.

A prompt takes what budget is left and continues next step (chunked prefill). With prefix
caching, a sequence starts with the pages of its leading full blocks that some earlier request
already computed, and publishes its own full blocks after every step.

Pure bookkeeping on sequences and the cache manager: no tensors.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from atomserve_b200.cache.manager import CacheManager
from atomserve_b200.config.engine_config import EngineConfig
from atomserve_b200.engine.sequence import Sequence, SequenceStatus, StepResult


@dataclass
class SchedulerOutput:
    """The plan for one step: seqs[i] runs its next num_new_tokens[i] tokens; `preempted`
    were evicted to make room and wait again."""

    seqs: list[Sequence] = field(default_factory=list)
    num_new_tokens: list[int] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(self.num_new_tokens)


class Scheduler:
    def __init__(self, config: EngineConfig, cache: CacheManager, eos_token_ids: frozenset[int] = frozenset()):
        self.config, self.cache, self.eos_token_ids = config, cache, frozenset(eos_token_ids)
        self.prefix_caching = config.enable_prefix_caching and cache.supports_prefix_caching
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []  # in admission order

    def add(self, seq: Sequence) -> None:
        if seq.cache is None:
            seq.cache = self.cache.new_request()
        self.waiting.append(seq)

    @property
    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    def schedule(self) -> SchedulerOutput:
        budget = self.config.max_num_batched_tokens
        out = SchedulerOutput()

        for seq in list(self.running):  # a copy: preemption shrinks the list
            if seq.status is not SequenceStatus.RUNNING:
                continue  # preempted earlier in this loop
            n = len(seq.token_ids) - seq.num_computed_tokens
            if n > budget:
                n = budget
            if n == 0:
                continue  # budget spent; it waits for the next step
            while not self.cache.reserve(seq.cache, seq.num_computed_tokens, n):
                victim = self.running[-1]  # newest: it has the least to redo
                self._preempt(victim)
                out.preempted.append(victim)
                if victim is seq:
                    break
            if seq.status is SequenceStatus.RUNNING:
                out.seqs.append(seq)
                out.num_new_tokens.append(n)
                budget -= n

        while self.waiting and not out.preempted and len(self.running) < self.config.max_num_seqs:
            seq = self.waiting[0]
            if self.prefix_caching:
                seq.num_computed_tokens = self.cache.use_cached_prefix(seq.cache, seq.token_ids)
                if not seq.output_ids:  # count hits on the prompt, not on redoing a preempted reply
                    seq.num_cached_tokens = seq.num_computed_tokens
            n = min(seq.num_tokens - seq.num_computed_tokens, budget)
            if n == 0 or not self.cache.admit(seq.cache) or not self.cache.reserve(seq.cache, seq.num_computed_tokens, n):
                self.cache.free(seq.cache)  # undo a prefix hit and the slot; retry next step
                seq.num_computed_tokens = seq.num_cached_tokens = 0
                break
            self.waiting.popleft()
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            out.seqs.append(seq)
            out.num_new_tokens.append(n)
            budget -= n
        return out

    def update(self, out: SchedulerOutput, results: list[StepResult]) -> list[tuple[Sequence, list[int]]]:
        """Apply a finished step; returns (sequence, its new tokens) for every sequence that
        got any. A finished sequence has only the tokens up to its stop."""
        new_tokens = []
        for seq, result in zip(out.seqs, results, strict=True):
            appended = []
            for token in result.tokens:
                seq.token_ids.append(token)
                appended.append(token)
                reason = self._finish_reason(seq, token)
                if reason:
                    self._finish(seq, reason)
                    break
            if appended:
                new_tokens.append((seq, appended))
            if seq.status is SequenceStatus.FINISHED:
                continue
            # the newest token's keys and values come with the next step
            seq.num_computed_tokens = min(result.num_computed, len(seq.token_ids) - 1)
            if self.prefix_caching:
                self.cache.register_full_blocks(seq.cache, seq.token_ids, seq.num_computed_tokens)
        return new_tokens

    def abort(self, seq_id: int) -> Sequence | None:
        for seq in [*self.waiting, *self.running]:
            if seq.id == seq_id:
                if seq in self.waiting:
                    self.waiting.remove(seq)
                self._finish(seq, "abort")
                return seq
        return None

    def _finish_reason(self, seq: Sequence, token: int) -> str | None:
        params, known = seq.params, len(seq.token_ids)
        if token in self.eos_token_ids and not params.ignore_eos:
            return "stop"
        if known - seq.num_prompt_tokens >= params.max_tokens or known >= self.config.max_model_len:
            return "length"
        return None

    def _preempt(self, seq: Sequence) -> None:
        self.running.remove(seq)
        self.cache.free(seq.cache)
        seq.num_computed_tokens = 0
        seq.status = SequenceStatus.WAITING
        self.waiting.appendleft(seq)

    def _finish(self, seq: Sequence, reason: str) -> None:
        if seq in self.running:
            self.running.remove(seq)
        if seq.cache is not None:
            self.cache.free(seq.cache)
        seq.status = SequenceStatus.FINISHED
        seq.finish_reason = reason
