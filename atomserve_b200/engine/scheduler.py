"""The scheduler: who runs in the next step, and how many tokens each.

Two limits bound a step: `max_num_seqs` sequences may hold cache at once, and
`max_num_batched_tokens` tokens may run at once. Within them a step is filled in two passes
(the policy is the reference's, atomserve/scheduler.py:1-35, 88-135):

  the resident pass   Every sequence that already holds cache gets its turn in the order it was
                      let in: a decoding one asks for one token, one still inside its prompt for
                      as much of the rest as the budget has left (so a long prompt is cut into
                      portions by whatever the decodes before it left over). If the cache cannot
                      give a sequence the pages it asks for, sequences are evicted from the young
                      end of the resident list until it can: an evicted sequence gives back all
                      it holds, goes to the front of the line and is computed again from its
                      tokens when it is let in next. The asker may end up evicting itself.
  the door pass       Skipped in a step that evicted anybody. Otherwise the line is served
                      strictly from its head while budget, the sequence limit, a state slot and
                      pages are there; the first sequence that does not fit stops the pass
                      (nobody overtakes it). With prefix caching a newcomer first takes over the
                      pages that hold its leading full blocks from some earlier request.

After the step, `update` appends what was sampled, retires what is done and, with prefix
caching, publishes the pages that became full.

Bookkeeping only: sequences and the cache manager, no tensors.
"""

from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from atomserve_b200.cache.manager import CacheManager
from atomserve_b200.config.engine_config import EngineConfig
from atomserve_b200.engine.sequence import Sequence, SequenceStatus, StepResult


@dataclass
class SchedulerOutput:
    """One step's plan: seqs[i] runs its next num_new_tokens[i] tokens. `preempted` lost their
    cache to make room and stand in line again."""

    seqs: list[Sequence] = field(default_factory=list)
    num_new_tokens: list[int] = field(default_factory=list)
    preempted: list[Sequence] = field(default_factory=list)

    @property
    def num_tokens(self) -> int:
        return sum(self.num_new_tokens)

    def grant(self, seq: Sequence, n: int) -> None:
        self.seqs.append(seq)
        self.num_new_tokens.append(n)


class Scheduler:
    def __init__(self, config: EngineConfig, cache: CacheManager, eos_token_ids: frozenset[int] = frozenset()):
        self.config, self.cache = config, cache
        self.eos_token_ids = frozenset(eos_token_ids)
        self.prefix_caching = config.enable_prefix_caching and cache.supports_prefix_caching
        self.waiting: deque[Sequence] = deque()  # the line, head first
        self.running: list[Sequence] = []  # residents, in the order they were let in
        self._known: dict[int, Sequence] = {}  # by request id, while waiting or resident

    # ---- arrivals and departures ---------------------------------------------------------------

    def add(self, seq: Sequence) -> None:
        if seq.cache is None:
            seq.cache = self.cache.new_request()
        self._known[seq.id] = seq
        self.waiting.append(seq)

    @property
    def has_work(self) -> bool:
        return bool(self._known)

    def abort(self, seq_id: int) -> Sequence | None:
        """Retire a sequence wherever it stands; None if it is not (or no longer) here."""
        seq = self._known.get(seq_id)
        if seq is None:
            return None
        if seq.status is SequenceStatus.WAITING:
            self.waiting.remove(seq)
        self._retire(seq, "abort")
        return seq

    def _retire(self, seq: Sequence, reason: str) -> None:
        if seq.status is SequenceStatus.RUNNING:
            self.running.remove(seq)
        self._known.pop(seq.id, None)
        if seq.cache is not None:
            self.cache.free(seq.cache)
        seq.status, seq.finish_reason = SequenceStatus.FINISHED, reason

    def _evict_youngest(self) -> Sequence:
        """The resident let in last has the least to compute again: it gives everything back and
        goes to the head of the line."""
        victim = self.running.pop()
        self.cache.free(victim.cache)
        victim.num_computed_tokens = 0
        victim.status = SequenceStatus.WAITING
        self.waiting.appendleft(victim)
        return victim

    # ---- planning a step -----------------------------------------------------------------------

    def schedule(self) -> SchedulerOutput:
        plan = SchedulerOutput()
        left = self._resident_pass(plan, self.config.max_num_batched_tokens)
        if not plan.preempted:
            self._door_pass(plan, left)
        return plan

    def _resident_pass(self, plan: SchedulerOutput, budget: int) -> int:
        residents, reserve = self.running, self.cache.reserve
        granted, counts = plan.seqs.append, plan.num_new_tokens.append
        # Evictions only ever shorten the list behind the sequence whose turn it is (or remove that
        # sequence itself, which is then the last), so walking by index meets each survivor once.
        turn = 0
        while turn < len(residents):
            seq = residents[turn]
            turn += 1
            ask = len(seq.token_ids) - seq.num_computed_tokens
            if ask > budget:
                ask = budget
            if ask <= 0:
                continue  # the budget is spent: it keeps what it holds and waits a step
            while not reserve(seq.cache, seq.num_computed_tokens, ask):
                victim = self._evict_youngest()
                plan.preempted.append(victim)
                if victim is seq:
                    break
            else:
                granted(seq)
                counts(ask)
                budget -= ask
        return budget

    def _door_pass(self, plan: SchedulerOutput, budget: int) -> None:
        line, cache = self.waiting, self.cache
        while line and len(self.running) < self.config.max_num_seqs:
            seq = line[0]
            have = 0
            if self.prefix_caching:
                have = cache.use_cached_prefix(seq.cache, seq.token_ids)
                # a hit counts for the prompt only, not for recomputing an evicted reply
                seq.num_cached_tokens = have if len(seq.token_ids) == seq.num_prompt_tokens else seq.num_cached_tokens
            ask = min(len(seq.token_ids) - have, budget)
            if ask <= 0 or not cache.admit(seq.cache) or not cache.reserve(seq.cache, have, ask):
                cache.free(seq.cache)  # gives back prefix pages and the slot, if it got that far
                seq.num_computed_tokens = seq.num_cached_tokens = 0
                return  # it stays at the head; nobody behind it is tried
            line.popleft()
            seq.num_computed_tokens = have
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            plan.grant(seq, ask)
            budget -= ask

    # ---- after a step --------------------------------------------------------------------------

    def update(self, out: SchedulerOutput, results: list[StepResult]) -> list[tuple[Sequence, list[int]]]:
        """Book a finished step. Returns (sequence, tokens it gained) for each sequence that gained
        any; a sequence that stops keeps nothing after its stopping token."""
        gained: list[tuple[Sequence, list[int]]] = []
        limit = self.config.max_model_len
        for seq, result in zip(out.seqs, results, strict=True):
            if seq.status is SequenceStatus.FINISHED:
                continue  # retired while its step was on the device (a step launched ahead, an abort): the row is dropped
            taken = 0
            reason = None
            for token in result.tokens:
                seq.token_ids.append(token)
                taken += 1
                reason = self._why_stop(seq, token, limit)
                if reason is not None:
                    break
            if taken:
                gained.append((seq, result.tokens[:taken]))
            if reason is not None:
                self._retire(seq, reason)
                continue
            # the newest token has no keys and values yet: they come with the step that feeds it
            seq.num_computed_tokens = min(result.num_computed, len(seq.token_ids) - 1)
            if self.prefix_caching:
                self.cache.register_full_blocks(seq.cache, seq.token_ids, seq.num_computed_tokens)
        return gained

    def _why_stop(self, seq: Sequence, token: int, limit: int) -> str | None:
        """"stop" on an end-of-sequence token (unless ignored), "length" when the reply or the
        whole sequence is as long as allowed (atomserve/scheduler.py:167-176)."""
        if token in self.eos_token_ids and not seq.params.ignore_eos:
            return "stop"
        total = len(seq.token_ids)
        if total - seq.num_prompt_tokens >= seq.params.max_tokens or total >= limit:
            return "length"
        return None
