"""Scheduler, cache manager, runner and engine together on the CPU, with the tests' torch parts
standing where the CUDA kernels are (tests/toy_parts.py): greedy tokens must equal the plain
implementation's under batching, chunking, preemption, prefix reuse and a window
(the reference's tests/test_engine.py:21-96 in this engine's terms)."""

import threading

import pytest
import torch

import plain_qwen3 as plain
import toy_parts
from atomserve_b200.cache import CacheManager
from atomserve_b200.config import EngineConfig
from atomserve_b200.engine.engine import Engine
from atomserve_b200.engine.runner import ModelRunner, Row
from atomserve_b200.engine.scheduler import Scheduler
from atomserve_b200.engine.sequence import SamplingParams
from helpers import checkpoint, prompts
from tiny_configs import TINY

GREEDY = dict(temperature=0.0, ignore_eos=True)


def widen(w):
    """Larger matrices so that greedy tokens vary instead of repeating one id."""
    return {k: (v * 6 if v.dim() == 2 else v) for k, v in w.items()}


@pytest.fixture(scope="module", params=["a", "b", "c"])
def setup(request):
    cfg, bs = TINY[request.param]
    w = widen(checkpoint(cfg, seed=8, sharp=False, bf16_exact=False))
    return cfg, bs, w, toy_parts.toy_model(cfg, w)


def engine_for(model, bs, **kw):
    config = EngineConfig(**{"block_size": bs, "num_blocks": 64, "max_model_len": 64 * bs, "max_num_seqs": 8,
                             "max_num_batched_tokens": 256, **kw})  # fmt: skip
    cache = CacheManager(model.cache_requirements(), bs, config.num_blocks, config.max_num_seqs, torch.float32, "cpu")
    return Engine(ModelRunner(model, cache), Scheduler(config, cache), toy_parts.ArgmaxSampler())


def test_step_function_matches_the_oracle_in_a_mixed_batch(setup):
    cfg, bs, w, model = setup
    cache = CacheManager(model.cache_requirements(), bs, 32, 4, torch.float32, "cpu")
    runner = ModelRunner(model, cache)
    a, b = prompts(cfg, [29, 11], seed=1)
    ra, rb = cache.new_request(), cache.new_request()
    cache.admit(ra), cache.admit(rb)
    cache.reserve(ra, 0, 20)
    first = runner.step([Row(a[:20], 0, ra, [0, 19])])
    cache.reserve(ra, 20, 9), cache.reserve(rb, 0, 11)
    second = runner.step([Row(a[20:], 20, ra, list(range(9))), Row(b, 0, rb, [10, 3])])
    oa, ob = plain.forward(w, cfg, a), plain.forward(w, cfg, b)
    assert torch.allclose(first, oa[[0, 19]], atol=2e-4)
    assert torch.allclose(second[:9], oa[20:], atol=2e-4)
    assert torch.allclose(second[9:], ob[[10, 3]], atol=2e-4)


def test_decode_steps_pack_the_block_tables_of_whoever_holds_the_slot(setup):
    """Steps of single tokens gather their block tables from a matrix kept per state slot: it has
    to follow tables that grow, a slot that passes to another request, a request that is freed
    and starts again, and requests that skip steps."""
    import random

    cfg, bs, w, model = setup
    cache = CacheManager(model.cache_requirements(), bs, 64, 3, torch.float32, "cpu")
    runner = ModelRunner(model, cache, cuda_graphs=False)
    rng = random.Random(3)
    live = {}  # uid -> [request, tokens held]
    for step in range(120):
        if len(live) < 3 and rng.random() < 0.5:
            rc = cache.new_request()
            assert cache.admit(rc)
            n = rng.randint(1, 3 * bs)
            assert cache.reserve(rc, 0, n)
            runner.step([Row([1] * n, 0, rc, [])])  # a prompt portion: the general path
            live[rc.uid] = [rc, n]
        if live and rng.random() < 0.15:
            rc = live.pop(rng.choice(list(live)))[0]
            cache.free(rc)  # the slot goes back; the next request may get it
            if rng.random() < 0.5:  # the same request starts again
                assert cache.admit(rc) and cache.reserve(rc, 0, 2)
                runner.step([Row([2, 3], 0, rc, [])])
                live[rc.uid] = [rc, 2]
        rows = []
        for rc, held in live.values():
            if rng.random() < 0.8 and held + 1 < 12 * bs and cache.reserve(rc, held, 1):
                rows.append(Row([5], held, rc, [0]))
        if not rows:
            continue
        with torch.inference_mode():  # as inside ModelRunner.step
            ctx, groups, _ = runner.prepare(rows)
        for g, (slots, tables) in enumerate(groups):
            group = cache.groups[g]
            for i, r in enumerate(rows):
                table = r.cache.block_tables[g]
                first = cache.first_needed_block(group, r.start)
                needed = r.start // bs + 1
                assert tables[i, first:needed].tolist() == table[first:needed], (step, g, i)
                assert int(slots[i]) == table[r.start // bs] * bs + r.start % bs
        for r in rows:
            live[r.cache.uid][1] += 1


def test_runner_rejects_bad_rows(setup):
    cfg, bs, w, model = setup
    cache = CacheManager(model.cache_requirements(), bs, 8, 2, torch.float32, "cpu")
    runner = ModelRunner(model, cache)
    rc = cache.new_request()
    cache.reserve(rc, 0, 3)
    with pytest.raises(ValueError, match="at least one token"):
        runner.step([Row([], 0, rc, [])])
    with pytest.raises(ValueError, match="wanted places"):
        runner.step([Row([1, 2], 0, rc, [2])])
    with pytest.raises(ValueError, match="block table holds"):
        runner.step([Row(list(range(bs + 1)), 0, rc, [])])
    with pytest.raises(ValueError, match="token id"):
        runner.step([Row([cfg["vocab_size"]], 0, rc, [])])


def test_greedy_equals_plain_alone_batched_chunked(setup):
    cfg, bs, w, model = setup
    ps = prompts(cfg, [5, 17, 33], seed=3)
    expect = [plain.greedy_generate(w, cfg, p, 8) for p in ps]
    params = SamplingParams(max_tokens=8, **GREEDY)
    assert engine_for(model, bs).generate(ps, params) == expect  # batched
    for p, e in zip(ps, expect):
        assert engine_for(model, bs).generate([p], params) == [e]  # alone
    chunked = engine_for(model, bs, max_num_batched_tokens=8, max_num_seqs=4)
    assert chunked.generate(ps, params) == expect
    assert chunked.num_steps > 8 + 3


def test_preemption_under_few_pages_keeps_outputs(setup):
    cfg, bs, w, model = setup
    ps = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    n = bs + 8  # every request grows by at least a page, and the pool cannot hold all three
    expect = [plain.greedy_generate(w, cfg, p, n) for p in ps]
    eng = engine_for(model, bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    assert eng.generate(ps, SamplingParams(max_tokens=n, **GREEDY)) == expect
    assert eng.stats()["preemptions"] > 0 and eng.stats()["kv_blocks_used"] == 0


def test_prefix_cache_hits_equal_uncached(setup):
    cfg, bs, w, model = setup
    shared = prompts(cfg, [3 * bs + 2], seed=6)[0]
    ps = [shared + [1, 2, 3], shared + [4]]
    expect = [plain.greedy_generate(w, cfg, p, 6) for p in ps]
    eng = engine_for(model, bs)
    params = SamplingParams(max_tokens=6, **GREEDY)
    got = [eng.generate([p], params)[0] for p in ps]
    assert got == expect
    if eng.scheduler.prefix_caching:
        assert eng.stats()["cached_prompt_tokens"] == 3 * bs
    else:
        assert cfg.get("use_sliding_window") and eng.stats()["cached_prompt_tokens"] == 0


def test_concurrent_clients_abort_and_validation(setup):
    cfg, bs, w, model = setup
    eng = engine_for(model, bs)
    with pytest.raises(ValueError, match="prompt has 0"):
        eng.submit([], SamplingParams())
    with pytest.raises(ValueError, match="max_tokens"):
        eng.submit([1], SamplingParams(max_tokens=0))
    with pytest.raises(ValueError, match="outside"):
        eng.submit([cfg["vocab_size"]], SamplingParams())
    eng.start()
    ps = prompts(cfg, [4, 9, 14, 6], seed=7)
    expect = [plain.greedy_generate(w, cfg, p, 5) for p in ps]
    results = [None] * 4

    def client(i):
        results[i] = list(eng.submit(ps[i], SamplingParams(max_tokens=5, **GREEDY)))

    threads = [threading.Thread(target=client, args=(i,)) for i in range(4)]
    [t.start() for t in threads]
    [t.join(timeout=120) for t in threads]
    assert results == expect
    handle = eng.submit(ps[2], SamplingParams(max_tokens=4000, **GREEDY))
    it = iter(handle)
    next(it)
    handle.abort()
    list(it)
    assert handle.finish_reason == "abort" and handle.ttft is not None
    eng.shutdown()
    assert eng.stats()["kv_blocks_used"] == 0 and eng.stats()["running"] == 0


def ahead_engine_for(model, bs, eos=frozenset(), **kw):
    config = EngineConfig(**{"block_size": bs, "num_blocks": 64, "max_model_len": 64 * bs, "max_num_seqs": 8,
                             "max_num_batched_tokens": 256, **kw})  # fmt: skip
    cache = CacheManager(model.cache_requirements(), bs, config.num_blocks, config.max_num_seqs, torch.float32, "cpu")
    return Engine(ModelRunner(model, cache), Scheduler(config, cache, frozenset(eos)), toy_parts.TwoPhaseArgmaxSampler())


def test_steps_launched_ahead_change_no_token(setup):
    """With a sampler that can start a step's sampling and be read later, the engine launches a
    decode-only step before it has read the step before it. The tokens must be those of the plain
    implementation: batched with different lengths (sequences ending by length at different
    steps), with end-of-sequence tokens that end sequences while the step ahead is on its way
    (its row is dropped), with so few pages that sequences are preempted, with a prefix shared."""
    cfg, bs, w, model = setup
    ps = prompts(cfg, [5, 17, 33, 2], seed=3)
    lengths = [9, 3, 14, 6]
    expect = [plain.greedy_generate(w, cfg, p, n) for p, n in zip(ps, lengths)]
    eng = ahead_engine_for(model, bs)
    handles = [eng.submit(p, SamplingParams(max_tokens=n, **GREEDY)) for p, n in zip(ps, lengths)]
    while eng.step():
        pass
    assert [list(h) for h in handles] == expect and [h.finish_reason for h in handles] == ["length"] * 4
    assert eng.stats()["steps_ahead"] >= 5 and eng.stats()["kv_blocks_used"] == 0
    # end-of-sequence tokens: whatever the third and the fifth token of the first reply are
    long = [plain.greedy_generate(w, cfg, p, 12) for p in ps]
    eos = {long[0][2], long[0][4]}
    def cut(out):
        for i, t in enumerate(out):
            if t in eos:
                return out[: i + 1]
        return out
    eng = ahead_engine_for(model, bs, eos=eos)
    got = eng.generate(ps, SamplingParams(max_tokens=12, temperature=0.0))
    assert got == [cut(o) for o in long] and len(got[0]) <= 3
    assert eng.stats()["steps_ahead"] > 0 and eng.stats()["kv_blocks_used"] == 0
    # few pages: preemption between steps launched ahead
    ps3 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    n = bs + 8
    eng = ahead_engine_for(model, bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    assert eng.generate(ps3, SamplingParams(max_tokens=n, **GREEDY)) == [plain.greedy_generate(w, cfg, p, n) for p in ps3]
    assert eng.stats()["preemptions"] > 0 and eng.stats()["steps_ahead"] > 0 and eng.stats()["kv_blocks_used"] == 0
    # a shared prefix, one request after the other on one engine
    shared = prompts(cfg, [3 * bs + 2], seed=6)[0]
    eng = ahead_engine_for(model, bs)
    for p in (shared + [1, 2, 3], shared + [4]):
        assert eng.generate([p], SamplingParams(max_tokens=6, **GREEDY)) == [plain.greedy_generate(w, cfg, p, 6)]


def test_abort_and_arrival_while_a_step_is_ahead(setup):
    """A request aborted while a step launched ahead still carries its row, and a request that
    arrives meanwhile: the others' tokens stay those of the plain implementation."""
    cfg, bs, w, model = setup
    ps = prompts(cfg, [7, 12, 20], seed=9)
    expect = [plain.greedy_generate(w, cfg, p, 10) for p in ps]
    eng = ahead_engine_for(model, bs)
    params = SamplingParams(max_tokens=10, **GREEDY)
    a, b = eng.submit(ps[0], params), eng.submit(ps[1], params)
    for _ in range(4):
        assert eng.step()
    assert eng._ahead is not None  # a step is on its way with rows of both
    b.abort()
    c = eng.submit(ps[2], params)
    while eng.step():
        pass
    assert list(a) == expect[0] and list(c) == expect[2]
    got_b = list(b)
    assert b.finish_reason == "abort" and 0 < len(got_b) < 10 and got_b == expect[1][: len(got_b)]
    assert eng.stats()["kv_blocks_used"] == 0 and eng.stats()["running"] == 0


def test_engine_survives_a_failing_step(setup):
    cfg, bs, w, model = setup
    eng = engine_for(model, bs)
    real = eng.execute
    eng.execute = lambda out: (_ for _ in ()).throw(RuntimeError("boom"))
    eng.start()
    handle = eng.submit([1, 2], SamplingParams(max_tokens=3, **GREEDY))
    with pytest.raises(RuntimeError, match="engine step failed"):
        list(handle)
    assert handle.finish_reason == "error"
    eng.execute = real
    again = eng.submit([1, 2], SamplingParams(max_tokens=3, **GREEDY))
    assert list(again) == plain.greedy_generate(w, cfg, [1, 2], 3)
    eng.shutdown()
    assert eng.stats()["kv_blocks_used"] == 0


def test_a_fault_reported_by_the_device_fails_the_step_and_not_the_engine(setup):
    """The engine looks at the device's status words after every step: a kernel that gave up a
    wait must not have its logits sampled and streamed as if nothing had happened."""
    from atomserve_b200.engine.engine import DeviceFault

    class Status:  # what ops.status.DeviceStatus offers the engine
        def __init__(self):
            self.sent, self.fault = 0, None

        def send_to_host(self):
            self.sent += 1

        def problem_on_host(self):
            fault, self.fault = self.fault, None
            return fault

    cfg, bs, w, model = setup
    eng = engine_for(model, bs)
    status = eng.runner.device_status = Status()
    status.fault = "a tcgen05 kernel gave up a bounded wait (GEMM: MMA issue)"
    eng.start()
    handle = eng.submit([1, 2], SamplingParams(max_tokens=3, **GREEDY))
    with pytest.raises(RuntimeError, match="engine step failed") as caught:
        list(handle)
    assert isinstance(caught.value.__cause__, DeviceFault) and "MMA issue" in str(caught.value.__cause__)
    assert handle.finish_reason == "error" and handle.num_output_tokens == 0
    again = eng.submit([1, 2], SamplingParams(max_tokens=3, **GREEDY))
    assert list(again) == plain.greedy_generate(w, cfg, [1, 2], 3)
    eng.shutdown()
    assert status.sent == eng.num_steps + 1 and eng.stats()["kv_blocks_used"] == 0


def test_status_words_name_what_went_wrong_and_clear():
    from atomserve_b200.ops.status import DeviceStatus

    status = DeviceStatus(torch.device("cpu"))
    assert status.problem() is None and status.problem_on_host() is None
    status.pipeline.fill_(2)
    status.embedding.fill_(1)
    status.send_to_host()
    text = status.problem_on_host()
    assert "MMA issue" in text and "outside the vocabulary" in text
    assert status.problem() is None and status.problem_on_host() is None
    status.pipeline.fill_(14)
    assert "prefill attention" in status.problem() and status.words.tolist() == [0, 0, 0, 0]


def test_a_mixer_whose_pages_hold_one_tensor():
    """The cache manager builds its pools from the tensors a mixer's PageSpec lists: here one
    narrow latent per token instead of keys and values, beside an ordinary attention layer (two
    groups, two kinds of pages). Whole, cut into portions and against the mixer's longhand."""
    from atomserve_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec, build_model

    cfg, bs = TINY["a"]
    d, eps, hd, rank = cfg["hidden_size"], cfg["rms_norm_eps"], cfg["head_dim"], 12
    w = checkpoint(cfg, seed=14, bf16_exact=False)
    g = torch.Generator().manual_seed(4)
    for n, shape in (("down", (rank, d)), ("query", (rank, d)), ("up", (d, rank))):
        w[f"model.layers.1.latent.{n}.weight"] = torch.randn(shape, generator=g) * 0.3
    attn = PartSpec("torch_attention", dict(num_heads=4, num_kv_heads=2, head_dim=hd, eps=eps, theta=cfg["rope_theta"]),
                    "model.layers.0.self_attn.")  # fmt: skip
    layers = []
    for i, mixer in enumerate([attn, PartSpec("latent_mixer", dict(rank=rank), "model.layers.1.latent.")]):
        p = f"model.layers.{i}."
        layers.append(LayerSpec("pre_norm", mixer, PartSpec("torch_swiglu", dict(intermediate_size=cfg["intermediate_size"]), p + "mlp."),
                                PartSpec("torch_rms_norm", dict(eps=eps), p + "input_layernorm."),
                                PartSpec("torch_rms_norm", dict(eps=eps), p + "post_attention_layernorm.")))  # fmt: skip
    spec = ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], max_positions=512,
                     embedding=PartSpec("torch_embedding", dict(vocab_size=cfg["vocab_size"]), "model.embed_tokens."),
                     layers=tuple(layers), schedule=(LayerCall(0), LayerCall(1)),
                     final_norm=PartSpec("torch_rms_norm", dict(eps=eps), "model.norm."),
                     head=PartSpec("torch_head", dict(vocab_size=cfg["vocab_size"], tied=True), "lm_head."))  # fmt: skip
    model = build_model(spec)
    wanted = {s.name for s in model.tensor_specs()}
    model.load({k: v for k, v in w.items() if k in wanted})
    requirements = model.cache_requirements()
    cache = CacheManager(requirements, bs, 16, 4, torch.float32, "cpu")
    assert [sorted(g.pools) for g in cache.groups] == [["k", "v"], ["latent"]]
    assert cache.groups[1].pools["latent"].shape == (1, 16, 1, bs, rank)
    assert CacheManager.bytes_per_block(requirements, bs, torch.float32) == (2 * 2 * hd + rank) * bs * 4
    assert not cache.supports_prefix_caching  # two groups
    ids = prompts(cfg, [37], seed=2)[0]
    results = []
    for portions in ([37], [5, 2, 13, 1, 1, 15]):
        cache = CacheManager(requirements, bs, 16, 4, torch.float32, "cpu")
        runner = ModelRunner(model, cache)
        rc = cache.new_request()
        cache.admit(rc)
        at, got = 0, []
        for n in portions:
            assert cache.reserve(rc, at, n)
            got.append(runner.step([Row(ids[at : at + n], at, rc, list(range(n)))]))
            at += n
        results.append(torch.cat(got))
        cache.free(rc)
        assert all(g.allocator.num_free == 16 for g in cache.groups)
    assert torch.allclose(results[0], results[1], atol=1e-5)
    mixer = model.blocks[1].mixer
    h = torch.randn(11, d, generator=g)
    view = cache.entry_view(1)
    view.block_tables, view.slots = torch.tensor([[3]], dtype=torch.int32), torch.arange(3 * bs, 3 * bs + 11, dtype=torch.int32)
    ctx = type("Ctx", (), dict(host_q_lens=[11], host_pos_start=[0]))()
    y = mixer.forward(h, torch.zeros_like(h), ctx, view)
    ref = toy_parts.latent_mixer_reference(h, *(w[f"model.layers.1.latent.{n}.weight"] for n in ("down", "query", "up")))
    assert torch.allclose(y.double(), ref, atol=1e-5)
