"""The engine: the one thread that owns the device, and the mailboxes through which client
threads reach it.

Clients never touch scheduler, cache or device. They post mail (`_Submit`, `_Cancel`) and read
their request's `RequestHandle`, which the engine thread feeds with the token ids of each step
and, last, a closing record with the reason. The engine thread (or whoever calls `step()` in
its place) repeats:

    read the mail                               new requests join the line, cancelled ones leave
    plan   = scheduler.schedule()               who runs how many tokens (host only)
    logits = runner.step(rows of the plan)      one pass over the step's tokens
    ids    = sampler.sample(logits, ...)        reading them back is the step's one wait
    the device's status words are looked at     a kernel that gave up a wait fails the step
    scheduler.update(plan, results)             book tokens, retire what is done
    hand each request its new ids

While every resident request is decoding and nobody waits at the door, one step more is on the
device than has been read: before the wait for a step's ids, the step after it is planned (the
same requests, one token each), packed and launched, with the ids taken where the sampler left
them on the device. The host's work for a step then overlaps the step before it instead of
standing between two steps (batch 8 of the 8B shape: 1,905 to 1,973 tokens a second end to end,
the device alone doing 2,000). A request that ends on an end-of-sequence token, or is cancelled,
while such a step carries its row is retired as usual and the row's result dropped
(`EngineConfig.decode_lookahead`, `Engine._plan_ahead`).

It deals in token ids only. The programming interface is the reference's
(atomserve/engine.py:41-264): `create_engine`, `Engine.submit / abort / start / shutdown /
generate / step / stats`, and a handle that is iterated for ids and carries `finish_reason`,
`ttft`, `decode_tokens_per_s` and `num_cached_tokens`.
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
from atomserve_b200.engine.runner import ModelRunner, Row, rows_for
from atomserve_b200.engine.scheduler import Scheduler, SchedulerOutput
from atomserve_b200.engine.sequence import SamplingParams, Sequence, SequenceStatus, StepResult
from atomserve_b200.parts.model import DecoderModel
from atomserve_b200.sampling.sampler import Sampler

# ---- what travels between client threads and the engine thread ---------------------------------


@dataclass
class _Submit:
    seq: Sequence
    handle: "RequestHandle"


@dataclass
class _Cancel:
    request_id: int


class _Wake:
    """Mail with no content: it only ends a blocking read of the mailbox (shutdown)."""


@dataclass
class _Closing:
    """The last record a handle receives."""

    reason: str  # "stop", "length", "abort" or "error"
    error: BaseException | None = None


class RequestHandle:
    """A client's view of its request. Iterating it yields token ids as steps produce them and
    ends when the request does; the figures below are filled in by the engine thread."""

    def __init__(self, request_id: int, cancel, num_prompt_tokens: int):
        self.id = request_id
        self.num_prompt_tokens = num_prompt_tokens
        self.num_output_tokens = 0
        self.num_cached_tokens = 0  # prompt tokens that the prefix cache supplied
        self.finish_reason: str | None = None
        self.submitted_at = time.perf_counter()
        self.first_token_at: float | None = None
        self.finished_at: float | None = None
        self._cancel = cancel
        self._feed: queue.SimpleQueue = queue.SimpleQueue()  # lists of ids, then one _Closing

    def __iter__(self) -> Iterator[int]:
        while True:
            item = self._feed.get()
            if isinstance(item, _Closing):
                self.finish_reason = item.reason
                if item.error is not None:
                    raise RuntimeError("engine step failed") from item.error
                return
            yield from item

    def abort(self) -> None:
        self._cancel(self.id)

    @property
    def ttft(self) -> float | None:
        """Seconds from submission to the first token."""
        if self.first_token_at is None:
            return None
        return self.first_token_at - self.submitted_at

    @property
    def decode_tokens_per_s(self) -> float | None:
        """Tokens per second after the first one (None until the request has ended with two)."""
        if self.finished_at is None or self.first_token_at is None or self.num_output_tokens < 2:
            return None
        return (self.num_output_tokens - 1) / max(self.finished_at - self.first_token_at, 1e-9)

    # engine thread only
    def _deliver(self, tokens: list[int], now: float) -> None:
        if self.first_token_at is None:
            self.first_token_at = now
        self.num_output_tokens += len(tokens)
        self._feed.put(tokens)

    def _close(self, reason: str, error: BaseException | None, cached: int) -> None:
        self.num_cached_tokens = cached
        self.finished_at = time.perf_counter()
        self._feed.put(_Closing(reason, error))


class DeviceFault(RuntimeError):
    """A kernel reported through the device's status words that it could not finish its work;
    the step's logits are not to be trusted."""


class _Launched:
    """A step whose kernels are on the device and whose sampled ids have not been read yet."""

    __slots__ = ("plan", "reached", "wants", "picked")

    def __init__(self, plan: SchedulerOutput, reached: list[int], wants: list[bool], picked):
        self.plan, self.reached, self.wants, self.picked = plan, reached, wants, picked


class Engine:
    def __init__(self, runner: ModelRunner, scheduler: Scheduler, sampler: Sampler, lookahead: bool = True):
        self.runner, self.scheduler, self.sampler = runner, scheduler, sampler
        # One step may be in flight beyond the one being read (see `_plan_ahead`); it takes a
        # sampler that can start a step's sampling without waiting for it.
        self.lookahead = lookahead and hasattr(sampler, "launch") and hasattr(sampler, "collect")
        self._ahead: _Launched | None = None
        self._mail: queue.SimpleQueue = queue.SimpleQueue()
        self._open: dict[int, RequestHandle] = {}  # requests the scheduler still knows
        self._next_id = itertools.count()
        self._thread: threading.Thread | None = None
        self._stop = threading.Event()
        # counters, written by the engine thread
        self.num_steps = 0
        self.last_batch_seqs = self.last_batch_tokens = 0
        self.num_prompt_tokens = self.num_cached_prompt_tokens = 0
        self.num_generated_tokens = 0
        self.num_preemptions = 0
        self.num_steps_ahead = 0  # steps launched before their predecessor had been read

    # ---- for clients, from any thread ----------------------------------------------------------

    def submit(self, prompt_ids: list[int], params: SamplingParams) -> RequestHandle:
        """Post a request; its handle comes back at once. Bad requests are refused here, on the
        caller's thread, before they can reach a kernel."""
        longest = self.scheduler.config.max_model_len
        if not 0 < len(prompt_ids) < longest:
            raise ValueError(f"prompt has {len(prompt_ids)} tokens; must be 1 to {longest - 1}")
        if params.max_tokens < 1:
            raise ValueError("max_tokens must be at least 1")
        vocab = self.runner.model.spec.vocab_size
        if min(prompt_ids) < 0 or max(prompt_ids) >= vocab:
            raise ValueError(f"prompt holds a token id outside [0, {vocab})")
        rid = next(self._next_id)
        handle = RequestHandle(rid, self.abort, len(prompt_ids))
        self._mail.put(_Submit(Sequence(rid, list(prompt_ids), params), handle))
        return handle

    def abort(self, request_id: int) -> None:
        """Ask for a request to be dropped; harmless if it has ended already."""
        self._mail.put(_Cancel(request_id))

    def start(self) -> None:
        self._thread = threading.Thread(target=self._serve, name="atomserve-b200-engine", daemon=True)
        self._thread.start()

    def shutdown(self) -> None:
        """Let the engine thread finish the step it is in, then end it."""
        self._stop.set()
        self._mail.put(_Wake())
        if self._thread is not None:
            self._thread.join()

    def generate(self, prompts: list[list[int]], params: SamplingParams) -> list[list[int]]:
        """Blocking convenience for tests, benchmarks and the command line: post every prompt,
        step on this thread until nothing is left, return each prompt's ids. Posting all of them
        before the first step is what batches them (atomserve/engine.py:137-146)."""
        handles = [self.submit(p, params) for p in prompts]
        while self.step():
            pass
        return [list(h) for h in handles]

    def stats(self) -> dict:
        sched, cache = self.scheduler, self.scheduler.cache
        pages = cache.num_blocks
        held = pages - cache.num_free_blocks
        return {
            "running": len(sched.running),
            "waiting": len(sched.waiting),
            "kv_blocks_used": held,
            "kv_blocks_total": pages,
            "kv_usage": held / pages,
            "kv_blocks_cached": sum(g.allocator.num_cached for g in cache.groups),
            "steps": self.num_steps,
            "last_batch_seqs": self.last_batch_seqs,
            "last_batch_tokens": self.last_batch_tokens,
            "prompt_tokens": self.num_prompt_tokens,
            "cached_prompt_tokens": self.num_cached_prompt_tokens,
            "generated_tokens": self.num_generated_tokens,
            "preemptions": self.num_preemptions,
            "steps_ahead": self.num_steps_ahead,
        }

    # ---- the engine thread ---------------------------------------------------------------------

    def step(self) -> bool:
        """Plan, run and book one step. False when no request is left to work on."""
        try:
            return self._step()
        except BaseException:
            self._ahead = None  # a step that raised leaves nothing on its way to be read later
            raise

    def _step(self) -> bool:
        self._read_mail(wait=False)
        launched, self._ahead = self._ahead, None
        if launched is None:
            if not self.scheduler.has_work:
                return False
            plan = self.scheduler.schedule()
            self.num_preemptions += len(plan.preempted)
            if not plan.seqs:
                raise RuntimeError("scheduler has work but scheduled nothing")
            if not self.lookahead:
                launched = None
                results = self.execute(plan)
            else:
                launched = self._launch(plan)
        if launched is not None:
            plan = launched.plan
            following = self._plan_ahead(plan)
            if following is not None:
                # its input is this step's sampled ids, taken on the device; the host reads them below
                self._ahead = self._launch(following, launched.picked.device_ids)
                self.num_steps_ahead += 1
            results = self._collect(launched)
        self._check_device()
        gained = self.scheduler.update(plan, results)

        self.num_steps += 1
        self.last_batch_seqs, self.last_batch_tokens = len(plan.seqs), plan.num_tokens
        now = time.perf_counter()
        for seq, tokens in gained:
            self.num_generated_tokens += len(tokens)
            self._open[seq.id]._deliver(tokens, now)
            if seq.status is SequenceStatus.FINISHED:
                self._close(seq)
        return True

    def execute(self, plan: SchedulerOutput) -> list[StepResult]:
        """The device's part of a step: run the plan's rows and sample one token for every
        sequence whose row reaches the end of its known tokens (atomserve/runner.py:194-212)."""
        return self._collect(self._launch(plan))

    def _launch(self, plan: SchedulerOutput, device_tokens=None) -> _Launched:
        """Put a step's kernels on the device, sampling included, and wait for nothing. The status
        words are sent on their way to the host behind the model's kernels, so that the read of the
        sampled ids, the step's one wait, brings them along. With `device_tokens` the step is one
        launched ahead: every sequence brings the one token that its predecessor step has just
        sampled, which only the device knows yet."""
        if device_tokens is None:
            rows = rows_for(plan.seqs, plan.num_new_tokens)
            logits = self.runner.step(rows)
        else:
            rows = [Row([0], len(seq.token_ids), seq.cache, [0]) for seq in plan.seqs]
            logits = self.runner.step(rows, device_tokens)
        status = getattr(self.runner, "device_status", None)
        if status is not None:
            status.send_to_host()
        sampled = [seq for seq, row in zip(plan.seqs, rows) if row.want]
        if hasattr(self.sampler, "launch"):
            picked = self.sampler.launch(logits, sampled, 1 if device_tokens is not None else 0) if sampled else None
        else:
            picked = self.sampler.sample(logits, sampled)
        return _Launched(plan, [row.start + len(row.tokens) for row in rows], [bool(row.want) for row in rows], picked)

    def _collect(self, launched: _Launched) -> list[StepResult]:
        """Wait for a launched step's sampled ids (the step's one wait) and pair them with its rows."""
        picked = launched.picked
        if picked is not None and not isinstance(picked, list):
            picked = self.sampler.collect(picked)
        results, k = [], 0
        for reached, want in zip(launched.reached, launched.wants):
            if want:
                results.append(StepResult([picked[k]], reached))
                k += 1
            else:
                results.append(StepResult([], reached))
        return results

    def _plan_ahead(self, plan: SchedulerOutput) -> SchedulerOutput | None:
        """The step after `plan`, if it can be launched before `plan`'s tokens are read: `plan`
        is every resident sequence decoding one token, nobody waits at the door, no sequence ends
        with this token for its length (whether it ends on an end-of-sequence token only the read
        will tell: then the step ahead has computed one token too many for it, in pages that are
        the sequence's own until it is retired, and its row is dropped), none has a presence penalty
        (which needs the token on the host), and every sequence gets the page its next position
        needs. Then the following step is the same sequences, each with the token this step
        samples, and the host's work for it (rows, packing, launch) overlaps this step on the
        device instead of standing between two steps."""
        sched = self.scheduler
        if sched.waiting or plan.preempted or len(plan.seqs) != len(sched.running) or not self._mail.empty():
            return None
        limit = sched.config.max_model_len
        for seq, n in zip(plan.seqs, plan.num_new_tokens):
            have = len(seq.token_ids)
            if (n != 1 or seq.status is not SequenceStatus.RUNNING or seq.num_computed_tokens + 1 != have
                    or seq.params.presence_penalty != 0 or have + 1 >= limit
                    or have + 1 - seq.num_prompt_tokens >= seq.params.max_tokens):  # fmt: skip
                return None
        for seq in plan.seqs:
            if not sched.cache.reserve(seq.cache, len(seq.token_ids), 1):
                return None  # (what the others were given they keep: they need it next step anyway)
        following = SchedulerOutput()
        for seq in plan.seqs:
            following.grant(seq, 1)
        return following

    def _check_device(self) -> None:
        status = getattr(self.runner, "device_status", None)
        if status is not None:
            problem = status.problem_on_host()
            if problem:
                raise DeviceFault(problem)

    def _read_mail(self, wait: bool) -> None:
        """Move what clients posted into the scheduler; with `wait`, sleep until something comes."""
        while True:
            try:
                mail = self._mail.get(block=wait)
            except queue.Empty:
                return
            wait = False
            if isinstance(mail, _Submit):
                self._open[mail.seq.id] = mail.handle
                self.num_prompt_tokens += mail.seq.num_prompt_tokens
                self.scheduler.add(mail.seq)
            elif isinstance(mail, _Cancel):
                dropped = self.scheduler.abort(mail.request_id)
                if dropped is not None:
                    self._close(dropped)

    def _close(self, seq: Sequence, error: BaseException | None = None) -> None:
        handle = self._open.pop(seq.id)
        self.num_cached_prompt_tokens += seq.num_cached_tokens
        self.sampler.release(seq.id)
        handle._close(seq.finish_reason or "error", error, seq.num_cached_tokens)

    def _fail_everything(self, error: BaseException) -> None:
        """A step raised: every request the scheduler knows ends with reason "error" and gives its
        pages back; the engine itself carries on with whatever is submitted next."""
        sched = self.scheduler
        self._ahead = None
        for seq in [*sched.running, *sched.waiting]:
            sched.abort(seq.id)
            seq.finish_reason = "error"
            self._close(seq, error)

    def _serve(self) -> None:
        while not self._stop.is_set():
            try:
                if not self.step():
                    self._read_mail(wait=True)
            except Exception as error:  # noqa: BLE001  the requests fail, the engine lives on
                traceback.print_exc(file=sys.stderr)
                self._fail_everything(error)


def create_engine(
    model: DecoderModel,
    engine_config: EngineConfig,
    eos_token_ids: frozenset[int] = frozenset(),
    sampler_seed: int | None = None,
) -> Engine:
    """Cache pools, runner, scheduler and sampler around a loaded model; the engine thread is
    not started (atomserve/engine.py:237-264)."""
    c = engine_config
    cache = CacheManager(model.cache_requirements(), c.block_size, c.num_blocks, c.max_num_seqs, model.dtype, model.device)
    runner = ModelRunner(model, cache, c.cuda_graphs)
    return Engine(runner, Scheduler(c, cache, eos_token_ids), Sampler(model.device, sampler_seed), c.decode_lookahead)
