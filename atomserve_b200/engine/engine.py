"""The engine: one loop that owns the device and runs scheduled steps.

    loop:
        take new requests and aborts from the inbox    -> scheduler
        plan    = scheduler.schedule()                  what runs this step (host only)
        logits  = runner.step(rows of the plan)         one forward pass
        tokens  = sampler.sample(logits, ...)           the step's one synchronisation
        scheduler.update(plan, results)                 advance, retire finished requests
        push each new token to its request's handle

Clients talk to it through a thread-safe inbox and one outbox per request; it deals in token
ids only. The programming interface follows the reference's (atomserve/engine.py:41-264):
`create_engine`, `Engine.submit / abort / start / shutdown / generate / step / stats`, and
`RequestHandle` as an iterator of token ids with `finish_reason`, `ttft` and
`decode_tokens_per_s`.
"""

from __future__ import annotations

import itertools
import queue
import sys
import threading
import time
import traceback
from collections.abc import Iterator
from dataclasses import dataclass

from atomserve_b200.cache.manager import CacheManager
from atomserve_b200.config.engine_config import EngineConfig
from atomserve_b200.engine.runner import ModelRunner, rows_for
from atomserve_b200.engine.scheduler import Scheduler, SchedulerOutput
from atomserve_b200.engine.sequence import SamplingParams, Sequence, SequenceStatus, StepResult
from atomserve_b200.parts.model import DecoderModel
from atomserve_b200.sampling.sampler import Sampler


@dataclass
class _Finished:
    reason: str  # "stop", "length", "abort" or "error"
    error: BaseException | None = None


class RequestHandle:
    """The client's end of one request: iterate it to receive token ids as they are made."""

    def __init__(self, request_id: int, engine: "Engine", num_prompt_tokens: int):
        self.id = request_id
        self.num_prompt_tokens = num_prompt_tokens
        self.num_output_tokens = 0
        self.num_cached_tokens = 0
        self.finish_reason: str | None = None
        self.submitted_at = time.perf_counter()
        self.first_token_at: float | None = None
        self.finished_at: float | None = None
        self._engine = engine
        self._outbox: queue.SimpleQueue = queue.SimpleQueue()

    def __iter__(self) -> Iterator[int]:
        while True:
            event = self._outbox.get()
            if isinstance(event, _Finished):
                self.finish_reason = event.reason
                if event.error is not None:
                    raise RuntimeError("engine step failed") from event.error
                return
            yield event

    def abort(self) -> None:
        self._engine.abort(self.id)

    @property
    def ttft(self) -> float | None:
        return None if self.first_token_at is None else self.first_token_at - self.submitted_at

    @property
    def decode_tokens_per_s(self) -> float | None:
        if self.first_token_at is None or self.finished_at is None or self.num_output_tokens < 2:
            return None
        return (self.num_output_tokens - 1) / max(self.finished_at - self.first_token_at, 1e-9)


class Engine:
    def __init__(self, runner: ModelRunner, scheduler: Scheduler, sampler: Sampler):
        self.runner, self.scheduler, self.sampler = runner, scheduler, sampler
        self._inbox: queue.SimpleQueue = queue.SimpleQueue()
        self._handles: dict[int, RequestHandle] = {}
        self._ids = itertools.count()
        self._thread: threading.Thread | None = None
        self._stopping = False
        self.num_steps = 0
        self.last_batch_seqs = 0
        self.last_batch_tokens = 0
        self.num_prompt_tokens = 0
        self.num_cached_prompt_tokens = 0
        self.num_generated_tokens = 0
        self.num_preemptions = 0

    # ---- client side (any thread) ---------------------------------------------------------------

    def submit(self, prompt_ids: list[int], params: SamplingParams) -> RequestHandle:
        limit = self.scheduler.config.max_model_len
        if not 0 < len(prompt_ids) < limit:
            raise ValueError(f"prompt has {len(prompt_ids)} tokens; must be 1 to {limit - 1}")
        if params.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        vocab = self.runner.model.spec.vocab_size
        if min(prompt_ids) < 0 or max(prompt_ids) >= vocab:
            raise ValueError(f"prompt holds a token id outside [0, {vocab})")
        request_id = next(self._ids)
        handle = RequestHandle(request_id, self, len(prompt_ids))
        self._inbox.put(("add", Sequence(request_id, list(prompt_ids), params), handle))
        return handle

    def abort(self, request_id: int) -> None:
        self._inbox.put(("abort", request_id))

    def start(self) -> None:
        self._thread = threading.Thread(target=self._loop, name="atomserve-b200-engine", daemon=True)
        self._thread.start()

    def shutdown(self) -> None:
        self._stopping = True
        self._inbox.put(("wake",))
        if self._thread is not None:
            self._thread.join()

    def generate(self, prompts: list[list[int]], params: SamplingParams) -> list[list[int]]:
        """Run prompts to completion on the calling thread; each one's output ids. All are
        submitted first, so they are batched together (atomserve/engine.py:137-146)."""
        handles = [self.submit(p, params) for p in prompts]
        while self.step():
            pass
        return [list(h) for h in handles]

    def stats(self) -> dict:
        s = self.scheduler
        total = s.cache.num_blocks
        used = total - s.cache.num_free_blocks
        return {
            "running": len(s.running),
            "waiting": len(s.waiting),
            "kv_blocks_used": used,
            "kv_blocks_total": total,
            "kv_usage": used / total,
            "kv_blocks_cached": sum(g.allocator.num_cached for g in s.cache.groups),
            "steps": self.num_steps,
            "last_batch_seqs": self.last_batch_seqs,
            "last_batch_tokens": self.last_batch_tokens,
            "prompt_tokens": self.num_prompt_tokens,
            "cached_prompt_tokens": self.num_cached_prompt_tokens,
            "generated_tokens": self.num_generated_tokens,
            "preemptions": self.num_preemptions,
        }

    # ---- engine side (engine thread only) -------------------------------------------------------

    def execute(self, out: SchedulerOutput) -> list[StepResult]:
        """Run one scheduled step and sample: a sequence that reaches the end of its known
        tokens gets one new token (atomserve/runner.py:194-212)."""
        logits = self.runner.step(rows_for(out.seqs, out.num_new_tokens))
        ends = [s.num_computed_tokens + n == len(s.token_ids) for s, n in zip(out.seqs, out.num_new_tokens)]  # reaches_end
        sampled = iter(self.sampler.sample(logits, [s for s, end in zip(out.seqs, ends) if end]))
        return [
            StepResult([next(sampled)] if end else [], seq.num_computed_tokens + n)
            for seq, n, end in zip(out.seqs, out.num_new_tokens, ends)
        ]

    def step(self) -> bool:
        """One scheduling step; False when there is nothing to do."""
        self._drain_inbox(block=False)
        if not self.scheduler.has_work:
            return False
        out = self.scheduler.schedule()
        self.num_preemptions += len(out.preempted)
        if not out.seqs:
            raise RuntimeError("scheduler has work but scheduled nothing")
        results = self.execute(out)
        new_tokens = self.scheduler.update(out, results)

        now = time.perf_counter()
        self.num_steps += 1
        self.last_batch_seqs, self.last_batch_tokens = len(out.seqs), out.num_tokens
        for seq, tokens in new_tokens:
            handle = self._handles[seq.id]
            if handle.first_token_at is None:
                handle.first_token_at = now
            handle.num_output_tokens += len(tokens)
            self.num_generated_tokens += len(tokens)
            for token in tokens:
                handle._outbox.put(token)
            if seq.status is SequenceStatus.FINISHED:
                self._close(seq)
        return True

    def _drain_inbox(self, block: bool) -> None:
        while True:
            try:
                message = self._inbox.get(block=block)
            except queue.Empty:
                return
            block = False
            if message[0] == "add":
                _, seq, handle = message
                self._handles[seq.id] = handle
                self.num_prompt_tokens += seq.num_prompt_tokens
                self.scheduler.add(seq)
            elif message[0] == "abort":
                seq = self.scheduler.abort(message[1])
                if seq is not None:
                    self._close(seq)

    def _close(self, seq: Sequence, error: BaseException | None = None) -> None:
        handle = self._handles.pop(seq.id)
        handle.num_cached_tokens = seq.num_cached_tokens
        self.num_cached_prompt_tokens += seq.num_cached_tokens
        handle.finished_at = time.perf_counter()
        self.sampler.release(seq.id)
        handle._outbox.put(_Finished(seq.finish_reason or "error", error))

    def _loop(self) -> None:
        while not self._stopping:
            try:
                if not self.step():
                    self._drain_inbox(block=True)
            except Exception as error:  # noqa: BLE001  fail the requests, keep the engine alive
                traceback.print_exc(file=sys.stderr)
                for seq in [*self.scheduler.running, *self.scheduler.waiting]:
                    self.scheduler.abort(seq.id)
                    seq.finish_reason = "error"
                    self._close(seq, error)


def create_engine(
    model: DecoderModel,
    engine_config: EngineConfig,
    eos_token_ids: frozenset[int] = frozenset(),
    sampler_seed: int | None = None,
) -> Engine:
    """Wire cache pools, runner, scheduler and sampler around a loaded model (the thread is
    not started). atomserve/engine.py:237-264."""
    cache = CacheManager(
        model.cache_requirements(), engine_config.block_size, engine_config.num_blocks,
        engine_config.max_num_seqs, model.dtype, model.device,
    )  # fmt: skip
    runner = ModelRunner(model, cache, engine_config.cuda_graphs)
    return Engine(runner, Scheduler(engine_config, cache, eos_token_ids), Sampler(model.device, sampler_seed))
