"""The scheduler's decisions, without a model: budget, portions, admission, what happens when
pages run out, finish reasons, abort, prefix reuse. A fake runner simulates the cache slot by
slot and predicts each next token from what it reads back, so wrong sharing, a stale prefix or
a missing recomputation changes the output (the idea of the reference's
tests/test_scheduler.py:20-46)."""

import pytest

from atomserve_b200.cache import CacheManager
from atomserve_b200.config import EngineConfig
from atomserve_b200.engine.scheduler import Scheduler
from atomserve_b200.engine.sequence import SamplingParams, Sequence, SequenceStatus, StepResult
from atomserve_b200.parts import KVCacheSpec

SPEC = [(KVCacheSpec(1, 8, None), [])]


class FakeRunner:
    """Keeps one token id per cache slot; the 'model' sums the tokens it reads back through the
    block table, so the next token is right only if every earlier token sits where the table
    says."""

    def __init__(self, block_size):
        self.bs, self.slots = block_size, {}

    def execute(self, out):
        results = []
        for seq, n in zip(out.seqs, out.num_new_tokens):
            table, start = seq.cache.block_tables[0], seq.num_computed_tokens
            for p in range(start, start + n):
                self.slots[table[p // self.bs] * self.bs + p % self.bs] = seq.token_ids[p]
            tokens = []
            if seq.reaches_end(n):
                read = [self.slots[table[p // self.bs] * self.bs + p % self.bs] for p in range(start + n)]
                assert read == seq.token_ids, "the cache does not hold this sequence's tokens"
                tokens = [expected_next(read)]
            results.append(StepResult(tokens, start + n))
        return results


def expected_next(tokens):
    return (sum(tokens) * 31 + len(tokens)) % 1000


def expected_output(prompt, n):
    ids = list(prompt)
    for _ in range(n):
        ids.append(expected_next(ids))
    return ids[len(prompt):]


def make(num_blocks=64, block_size=4, **kw):
    config = EngineConfig(block_size=block_size, num_blocks=num_blocks,
                          **{"max_model_len": min(256, num_blocks * block_size), "max_num_seqs": 8,
                             "max_num_batched_tokens": 64, **kw})  # fmt: skip
    cache = CacheManager(SPEC, block_size, num_blocks, config.max_num_seqs)
    return Scheduler(config, cache, frozenset({999})), FakeRunner(block_size)


def seq(i, prompt, **params):
    return Sequence(i, list(prompt), SamplingParams(**{"max_tokens": 8, **params}))


def run(s, runner, limit=10000):
    plans = []
    while s.has_work:
        out = s.schedule()
        assert out.seqs, "work but nothing scheduled"
        s.update(out, runner.execute(out))
        check_invariants(s)
        plans.append(out)
        assert len(plans) < limit
    return plans


def check_invariants(s):
    alloc = s.cache.groups[0].allocator
    held = {}
    for q in s.running:
        assert q.status is SequenceStatus.RUNNING and q.cache.state_slot >= 0
        for b in q.cache.block_tables[0]:
            held[b] = held.get(b, 0) + 1
    for q in s.waiting:
        assert q.cache.block_tables == [[]] and q.cache.state_slot == -1
    for b in range(alloc.num_blocks):
        assert alloc.refcount(b) == held.get(b, 0)
    assert alloc.num_free == alloc.num_blocks - len(held)  # no page leaked
    assert len(s.running) <= s.config.max_num_seqs


def test_outputs_are_right_alone_and_batched():
    prompts = [[1, 2, 3], list(range(10, 27)), [7] * 9]
    s, r = make()
    seqs = [seq(i, p) for i, p in enumerate(prompts)]
    for q in seqs:
        s.add(q)
    run(s, r)
    for q, p in zip(seqs, prompts):
        assert q.output_ids == expected_output(p, 8) and q.finish_reason == "length"
    assert s.cache.num_free_blocks == 64


def test_budget_admission_and_portions():
    """A 20-token prompt under a budget of 8 beside one running decode runs as 7, 7, 6
    (the reference's tests/test_scheduler.py:152-170)."""
    s, r = make(max_num_batched_tokens=8, enable_prefix_caching=False)
    first = seq(0, [5, 6], max_tokens=20)
    s.add(first)
    out = s.schedule()
    s.update(out, r.execute(out))
    long = seq(1, range(100, 120), max_tokens=2)
    s.add(long)
    sizes = []
    for _ in range(3):
        out = s.schedule()
        assert out.seqs[0] is first and out.num_new_tokens[0] == 1  # running first
        sizes.append(out.num_new_tokens[1])
        results = r.execute(out)
        assert (results[1].tokens != []) == (len(sizes) == 3)  # a portion that stops short yields no token
        s.update(out, results)
    assert sizes == [7, 7, 6]


def test_head_of_line_is_not_skipped():
    s, r = make(num_blocks=6, max_model_len=24, enable_prefix_caching=False)
    s.add(seq(0, range(16), max_tokens=1))   # 4 pages
    s.add(seq(1, range(50, 66), max_tokens=1))  # needs 4: does not fit beside the first
    s.add(seq(2, [1], max_tokens=1))          # would fit, but must not overtake
    out = s.schedule()
    assert [q.id for q in out.seqs] == [0]
    assert [q.id for q in s.waiting] == [1, 2]


def test_pages_run_out_newest_is_preempted_and_recomputed():
    """Two sequences outgrow a pool of 6 pages: the newer one is evicted, everything it held is
    given back, it returns to the front of the queue and its output is still right."""
    s, r = make(num_blocks=6, max_model_len=24, enable_prefix_caching=False)
    a, b, c = seq(0, range(8), max_tokens=12), seq(1, range(20, 28), max_tokens=12), seq(2, [3], max_tokens=2)
    for q in (a, b):
        s.add(q)
    preempted = []
    steps = 0
    while s.has_work:
        out = s.schedule()
        if out.preempted and c.status is SequenceStatus.WAITING and c not in s.waiting:
            s.add(c)  # arrives while memory is short
        for victim in out.preempted:
            preempted.append(victim.id)
            assert victim.status is SequenceStatus.WAITING and victim.num_computed_tokens == 0
            assert s.waiting[0] is victim or victim in s.waiting
            assert victim not in out.seqs
        if out.preempted:
            assert all(q.num_computed_tokens > 0 or q in s.running for q in out.seqs)
            assert len(out.seqs) == len(s.running)  # nothing admitted in a step that preempted
        s.update(out, r.execute(out))
        check_invariants(s)
        steps += 1
        assert steps < 500
    assert preempted and preempted[0] == 1  # the newest running sequence goes first
    assert a.output_ids == expected_output(range(8), 12)
    assert b.output_ids == expected_output(range(20, 28), 12)
    assert c.output_ids == expected_output([3], 2)


def test_a_lone_sequence_that_needs_a_page_preempts_itself_and_still_finishes():
    s, r = make(num_blocks=4, max_model_len=16, enable_prefix_caching=False)
    a, b = seq(0, range(7), max_tokens=9), seq(1, range(30, 37), max_tokens=9)
    s.add(a)
    s.add(b)
    run(s, r)
    assert a.output_ids == expected_output(range(7), 9)  # reaches max_model_len 16 exactly
    assert b.output_ids == expected_output(range(30, 37), 9)


def test_finish_reasons():
    s, r = make()
    stop_at = expected_next([1, 2])
    s.eos_token_ids = frozenset({stop_at})
    a, b, c = seq(0, [1, 2]), seq(1, [1, 2], ignore_eos=True, max_tokens=3), seq(2, [4] * 250, max_tokens=50)
    for q in (a, b, c):
        s.add(q)
    run(s, r)
    assert a.finish_reason == "stop" and a.output_ids == [stop_at]
    assert b.finish_reason == "length" and len(b.output_ids) == 3
    assert c.finish_reason == "length" and c.num_tokens == 256  # max_model_len


def test_abort_frees_everything():
    s, r = make()
    a, b = seq(0, range(9), max_tokens=50), seq(1, range(5), max_tokens=50)
    s.add(a)
    out = s.schedule()
    s.update(out, r.execute(out))
    s.add(b)
    assert s.abort(0) is a and a.finish_reason == "abort" and a.status is SequenceStatus.FINISHED
    assert s.abort(1) is b and not s.has_work
    assert s.abort(7) is None
    assert s.cache.num_free_blocks == 64 and s.cache.state.num_free == 8


def test_sequence_limit_and_state_slots():
    s, r = make(max_num_seqs=2, max_num_batched_tokens=64)
    for i in range(5):
        s.add(seq(i, [i + 1] * 3, max_tokens=2))
    out = s.schedule()
    assert len(out.seqs) == 2 and len(s.waiting) == 3
    assert sorted(q.cache.state_slot for q in out.seqs) == [0, 1]
    s.update(out, r.execute(out))
    run(s, r)


def test_prefix_reuse_skips_shared_pages_and_stays_right():
    s, r = make()
    shared = list(range(40, 53))
    a = seq(0, shared + [1, 2], max_tokens=3)
    s.add(a)
    run(s, r)
    b = seq(1, shared + [9], max_tokens=3)
    s.add(b)
    out = s.schedule()
    assert b.num_cached_tokens == 12 and out.num_new_tokens == [2]  # three full pages of 4 reused
    s.update(out, r.execute(out))
    run(s, r)
    assert b.output_ids == expected_output(shared + [9], 3)
    # an identical prompt still computes its last token
    c = seq(2, shared + [1, 2], max_tokens=1)
    s.add(c)
    out = s.schedule()
    assert c.num_cached_tokens == 12 and out.num_new_tokens == [3]
    s.update(out, r.execute(out))
    assert c.output_ids == a.output_ids[:1]


def test_prefix_caching_is_off_for_windowed_or_stateful_models():
    from atomserve_b200.parts import StateSpec

    for reqs in ([(KVCacheSpec(1, 8, 16), [])], [(KVCacheSpec(1, 8, None), [StateSpec("s", (2,))])]):
        cache = CacheManager(reqs, 4, 16, 4)
        s = Scheduler(EngineConfig(block_size=4, num_blocks=16, max_model_len=64, max_num_seqs=4), cache)
        assert not s.prefix_caching
