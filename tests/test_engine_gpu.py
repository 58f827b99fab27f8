"""The engine on the GPU: greedy generation through the entry point, parts alone, run orders
that repeat a layer or share a cache, and a toy mixer with state of its own."""

import json
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as plain
import toy_parts
from helpers import FLOAT32_TOLERANCE, assert_near_best_tokens, checkpoint, prompts, rel_error, write_folder
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
GREEDY = dict(temperature=0.0, ignore_eos=True)


def widen(w):
    return {k: (v * 6 if v.dim() == 2 else v).bfloat16().float() if v.dim() == 2 else v for k, v in w.items()}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name, (cfg, bs) in TINY.items():
        w = widen(checkpoint(cfg, seed=8, sharp=False))
        out[name] = (cfg, bs, w, write_folder(cfg, w, tmp_path_factory.mktemp(f"gen_{name}")))
    return out


def engine_for(folder, dtype, bs, **kw):
    from atomserve_b200.config import EngineConfig
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.weights import load_model

    _, _, model = load_model(folder, dtype, "cuda")
    config = EngineConfig(**{"block_size": bs, "num_blocks": 64, "max_model_len": 64 * bs, "max_num_seqs": 8,
                             "max_num_batched_tokens": 256, **kw})  # fmt: skip
    return create_engine(model, config, sampler_seed=0)


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generation_float32_equals_plain(folders, name):
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, w, folder = folders[name]
    ps = prompts(cfg, [5, 17, 33], seed=3)
    expect = [plain.greedy_generate(w, cfg, p, 8) for p in ps]
    params = SamplingParams(max_tokens=8, **GREEDY)
    assert engine_for(folder, "float32", bs).generate(ps, params) == expect
    chunked = engine_for(folder, "float32", bs, max_num_batched_tokens=8, max_num_seqs=4)
    assert chunked.generate(ps, params) == expect
    short = engine_for(folder, "float32", bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    n = bs + 8
    ps2 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    assert short.generate(ps2, SamplingParams(max_tokens=n, **GREEDY)) == [plain.greedy_generate(w, cfg, p, n) for p in ps2]
    assert short.stats()["preemptions"] > 0 and short.stats()["kv_blocks_used"] == 0


@pytest.mark.parametrize("name", ["a", "b", "c"])
def test_greedy_generation_bfloat16_picks_near_best_tokens(folders, name):
    """bfloat16 may break near-ties differently, so each chosen token is judged against the
    oracle run on the engine's own sequence: its logit must lie within the bfloat16 allowance
    of the best."""
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, w, folder = folders[name]
    ps = prompts(cfg, [5, 17, 33], seed=3)
    outs = engine_for(folder, "bfloat16", bs).generate(ps, SamplingParams(max_tokens=8, **GREEDY))
    for p, out in zip(ps, outs):
        assert len(out) == 8
        assert_near_best_tokens(w, cfg, p, out, f"{name} batched")
    # in portions under a small budget, and with so few pages that requests are preempted
    chunked = engine_for(folder, "bfloat16", bs, max_num_batched_tokens=8, max_num_seqs=4)
    for p, out in zip(ps, chunked.generate(ps, SamplingParams(max_tokens=8, **GREEDY))):
        assert len(out) == 8
        assert_near_best_tokens(w, cfg, p, out, f"{name} chunked")
    assert chunked.num_steps > 8 + 3
    short = engine_for(folder, "bfloat16", bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    n = bs + 8
    ps2 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    for p, out in zip(ps2, short.generate(ps2, SamplingParams(max_tokens=n, **GREEDY))):
        assert len(out) == n
        assert_near_best_tokens(w, cfg, p, out, f"{name} preempted")
    assert short.stats()["preemptions"] > 0 and short.stats()["kv_blocks_used"] == 0


@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_prefix_cache_hits_on_the_gpu(folders, name):
    """Two prompts that share three full pages, one after the other through one engine: the
    second takes the first's pages (`cached_prompt_tokens`), and both get the plain
    implementation's tokens in float32; in bfloat16 tokens near the best."""
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, w, folder = folders[name]
    shared = prompts(cfg, [3 * bs + 2], seed=6)[0]
    ps = [shared + [1, 2, 3], shared + [4]]
    params = SamplingParams(max_tokens=6, **GREEDY)
    eng = engine_for(folder, "float32", bs)
    assert eng.scheduler.prefix_caching
    got = [eng.generate([p], params)[0] for p in ps]
    assert got == [plain.greedy_generate(w, cfg, p, 6) for p in ps]
    assert eng.stats()["cached_prompt_tokens"] == 3 * bs and eng.stats()["kv_blocks_cached"] >= 3
    eng = engine_for(folder, "bfloat16", bs)
    for p in ps:
        assert_near_best_tokens(w, cfg, p, eng.generate([p], params)[0], f"{name} prefix")
    assert eng.stats()["cached_prompt_tokens"] == 3 * bs


def test_four_client_threads_on_the_gpu(folders):
    """The engine thread owns the device; four client threads submit and iterate their handles
    (the reference's tests/test_engine.py:27-71 in this engine's terms); one request is aborted."""
    import threading

    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, w, folder = folders["b"]
    eng = engine_for(folder, "float32", bs)
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


def test_sampled_generation_is_seeded_and_in_support(folders):
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, w, folder = folders["b"]
    eng = engine_for(folder, "float32", bs)
    p = prompts(cfg, [12], seed=1)[0]
    params = SamplingParams(temperature=0.9, top_k=5, top_p=0.9, max_tokens=10, seed=11, ignore_eos=True)
    a = eng.generate([p], params)[0]
    other = SamplingParams(temperature=1.2, top_k=0, top_p=1.0, max_tokens=10, ignore_eos=True)
    hb = [eng.submit(q, other) for q in prompts(cfg, [7, 9], seed=2)]
    ha = eng.submit(p, params)
    while eng.step():
        pass
    assert list(ha) == a and all(len(list(h)) == 10 for h in hb)  # same draws among other requests
    ref = plain.forward(w, cfg, p + a)
    for i, token in enumerate(a):
        dist = plain.sampling_distribution(ref[len(p) + i - 1], 0.9, 5, 0.9)
        assert dist[token] > 0
    pen = SamplingParams(temperature=0.0, presence_penalty=100.0, max_tokens=12, ignore_eos=True)
    out = eng.generate([p], pen)[0]
    assert len(set(out)) == len(out)  # a large penalty never repeats a generated token


def test_steps_launched_ahead_give_the_same_tokens(folders):
    """Decode-only steps launched before the step before them has been read (their input the
    sampled ids as they lie on the device) against the engine that reads every step first:
    the same tokens for seeded sampling (the draw counters run one ahead), for greedy requests of
    different lengths, and with end-of-sequence ids that end requests while a step is ahead."""
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, w, folder = folders["b"]
    ps = prompts(cfg, [12, 5, 30, 2], seed=4)
    for dtype in ("float32", "bfloat16"):
        outs = {}
        for ahead in (False, True):
            eng = engine_for(folder, dtype, bs, decode_lookahead=ahead)
            hs = [eng.submit(p, SamplingParams(temperature=0.9, top_k=8, top_p=0.95, max_tokens=n, seed=3 + i, ignore_eos=True))
                  for i, (p, n) in enumerate(zip(ps, [14, 3, 9, 20]))]  # fmt: skip
            hs += [eng.submit(p, SamplingParams(temperature=0.0, max_tokens=n, ignore_eos=True)) for p, n in zip(ps, [6, 17, 2, 11])]
            while eng.step():
                pass
            outs[ahead] = [list(h) for h in hs]
            assert (eng.stats()["steps_ahead"] > 5) == ahead and eng.stats()["kv_blocks_used"] == 0
        assert outs[True] == outs[False], dtype
    greedy = plain.greedy_generate(w, cfg, ps[0], 12)
    eos = frozenset({greedy[3]})
    from atomserve_b200.config import EngineConfig
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.weights import load_model

    _, _, model = load_model(folder, "float32", "cuda")
    config = EngineConfig(block_size=bs, num_blocks=64, max_model_len=64 * bs, max_num_seqs=8, max_num_batched_tokens=256)
    eng = create_engine(model, config, eos_token_ids=eos, sampler_seed=0)
    got = eng.generate(ps[:3], SamplingParams(temperature=0.0, max_tokens=12))
    for p, g in zip(ps[:3], got):
        full = plain.greedy_generate(w, cfg, p, 12)
        cut = next((i + 1 for i, t in enumerate(full) if t in eos), 12)
        assert g == full[:cut]
    assert len(got[0]) <= 4 and eng.stats()["steps_ahead"] > 0 and eng.stats()["kv_blocks_used"] == 0


def test_first_token_sees_only_itself(folders):
    from atomserve_b200.engine.replay import TraceReplayer

    cfg, bs, w, folder = folders["b"]
    rp = TraceReplayer(folder, "float32", 64, bs)
    for token in (0, 3, cfg["vocab_size"] - 1):
        got = rp.step([dict(id=token, tokens=[token], want=[0])], end=[token]).cpu()
        assert rel_error(got, plain.forward(w, cfg, [token])) < FLOAT32_TOLERANCE
    two = rp.step([dict(id="t", tokens=[5, 9], want=[0, 1])], end=["t"]).cpu()
    assert rel_error(two, plain.forward(w, cfg, [5, 9])) < FLOAT32_TOLERANCE
    assert rel_error(two[:1], plain.forward(w, cfg, [5])) < FLOAT32_TOLERANCE


def test_command_line(folders, tmp_path):
    cfg, bs, w, folder = folders["a"]
    p = prompts(cfg, [6], seed=4)[0]
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    done = subprocess.run(
        [sys.executable, "-m", "atomserve_b200", str(folder), "--dtype", "fp32", "--kv-mem-gb", "0.01",
         "--block-size", str(bs), "--prompt-ids", ",".join(map(str, p)), "--temperature", "0", "--max-tokens", "6",
         "--ignore-eos"],
        capture_output=True, text=True, timeout=600, cwd=root,
    )  # fmt: skip
    assert done.returncode == 0, done.stderr[-2000:]
    record = json.loads(done.stdout.strip().splitlines()[-1])
    assert record["output_ids"] == plain.greedy_generate(w, cfg, p, 6) and record["finish_reason"] == "length"


# ---- parts alone ------------------------------------------------------------------------------


def step_context(q_lens, pos_starts, slots=None):
    from atomserve_b200.parts import StepContext

    T = sum(q_lens)
    starts = [0]
    for n in q_lens:
        starts.append(starts[-1] + n)
    positions = [p for n, s in zip(q_lens, pos_starts) for p in range(s, s + n)]
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")  # noqa: E731
    return StepContext(
        num_tokens=T, num_requests=len(q_lens), token_ids=i32([0] * T), positions=i32(positions),
        req_q_start=i32(starts), req_pos_start=i32(pos_starts), state_slots=i32(slots or list(range(len(q_lens)))),
        logits_rows=i32([]), max_context=max(s + n for n, s in zip(q_lens, pos_starts)),
        host_q_lens=list(q_lens), host_pos_start=list(pos_starts), host_state_slots=slots or list(range(len(q_lens))),
    )  # fmt: skip


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_attention_part_alone(dtype):
    """The mixer by itself, with sizes of its own: two portions of one sequence through its
    cache equal the plain attention block on the whole sequence."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, H, KV, hd, bs, T = 72, 6, 2, 48, 4, 23
    cfg = dict(num_attention_heads=H, num_key_value_heads=KV, head_dim=hd, rms_norm_eps=2e-6, rope_theta=3e4, hidden_size=d)
    g = torch.Generator().manual_seed(0)
    names = {"q_proj": (H * hd, d), "k_proj": (KV * hd, d), "v_proj": (KV * hd, d), "o_proj": (d, H * hd)}
    w = {f"x.self_attn.{n}.weight": (torch.randn(s, generator=g) * 0.1).bfloat16().float() for n, s in names.items()}
    w["x.self_attn.q_norm.weight"] = 1 + 0.1 * torch.randn(hd, generator=g)
    w["x.self_attn.k_norm.weight"] = 1 + 0.1 * torch.randn(hd, generator=g)
    part = build_part("mixer", PartSpec("gqa_attention", dict(
        num_heads=H, num_kv_heads=KV, head_dim=hd, qk_norm_eps=2e-6,
        position=PartSpec("rotary", dict(head_dim=hd, theta=3e4))), "x.self_attn."), d)  # fmt: skip
    part.load({k: v.cuda().to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()})
    h = torch.randn(T, d, generator=g).bfloat16().float()
    res = torch.randn(T, d, generator=g).bfloat16().float()
    ref = res + plain.attention_block(h, w, "x.", cfg, torch.arange(T), None)
    view = CacheView(k=torch.zeros(8, KV, bs, hd, device="cuda", dtype=dtype), block_size=bs)
    view.v = torch.zeros_like(view.k)
    table = [5, 2, 7, 0, 3, 6]
    view.block_tables = torch.tensor([table], dtype=torch.int32, device="cuda")
    outs = []
    for start, n in ((0, 14), (14, 9)):
        view.slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(start, start + n)], dtype=torch.int32, device="cuda")
        outs.append(part.forward(h[start : start + n].cuda().to(dtype), res[start : start + n].cuda().to(dtype),
                                 step_context([n], [start]), view))  # fmt: skip
    got = torch.cat(outs).float().cpu()
    assert rel_error(got, ref) < (1e-5 if dtype == torch.float32 else 2e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_norm_block_embedding_and_head_alone(dtype):
    from atomserve_b200.parts import PartSpec, build_part

    d, inter, T, V = 88, 200, 9, 77
    g = torch.Generator().manual_seed(1)
    w = {"m.mlp.gate_proj.weight": torch.randn(inter, d, generator=g) * 0.1, "m.mlp.up_proj.weight": torch.randn(inter, d, generator=g) * 0.1,
         "m.mlp.down_proj.weight": torch.randn(d, inter, generator=g) * 0.1}  # fmt: skip
    w = {k: v.bfloat16().float() for k, v in w.items()}
    ff = build_part("feed_forward", PartSpec("swiglu", dict(intermediate_size=inter), "m.mlp."), d)
    ff.load({k: v.cuda().to(dtype) for k, v in w.items()})
    h, res = (torch.randn(T, d, generator=g).bfloat16().float() for _ in range(2))
    got = ff.forward(h.cuda().to(dtype), res.cuda().to(dtype), None).float().cpu()
    assert rel_error(got, res + plain.swiglu_mlp(h, w, "m.")) < (1e-5 if dtype == torch.float32 else 2e-2)

    norm = build_part("norm", PartSpec("rms_norm", dict(eps=1e-4), "n."), d)
    gain = 1 + 0.1 * torch.randn(d, generator=g)
    norm.load({"n.weight": gain.cuda()})
    got = norm.forward(h.cuda().to(dtype)).float().cpu()
    assert rel_error(got, plain.rms_norm(h, gain, 1e-4)) < (1e-5 if dtype == torch.float32 else 1e-2)

    emb = build_part("embedding", PartSpec("token_embedding", dict(vocab_size=V), "e."), d)
    table = torch.randn(V, d, generator=g).bfloat16().float()
    emb.load({"e.weight": table.cuda().to(dtype)})
    ids = torch.tensor([0, V - 1, 5], dtype=torch.int32, device="cuda")
    assert torch.equal(emb.forward(ids).float().cpu(), table[[0, V - 1, 5]])
    head = build_part("head", PartSpec("lm_head", dict(vocab_size=V, tied=True), "lm_head."), d)
    head.tie(emb)
    logits = head.forward(h.cuda().to(dtype))
    assert logits.dtype == torch.float32 and rel_error(logits.cpu(), h @ table.T) < 1e-5


# ---- run orders and a mixer with state ----------------------------------------------------------


def custom_model(spec, w, device, dtype):
    from atomserve_b200.parts import build_model

    model = build_model(spec)
    model.load({k: v.to(device).to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()})
    return model


def run_whole_and_cut(model, bs, ids, cuts, device):
    """Logits of `ids` at every position: in one step, and cut into the given portions."""
    from atomserve_b200.cache import CacheManager
    from atomserve_b200.engine.runner import ModelRunner, Row

    results = []
    for portions in ([len(ids)], cuts):
        cache = CacheManager(model.cache_requirements(), bs, 32, 4, model.dtype, device)
        runner = ModelRunner(model, cache)
        rc = cache.new_request()
        cache.admit(rc)
        at, got = 0, []
        for n in portions:
            assert cache.reserve(rc, at, n)
            got.append(runner.step([Row(ids[at : at + n], at, rc, list(range(n)))]).float().cpu())
            at += n
        results.append(torch.cat(got))
    return results


def shared_cache_spec(cfg, kinds):
    """Four run-order entries over two layers: layer 0, layer 1, layer 0 again (a cache of its
    own), and layer 1 reading the cache that its first call wrote."""
    from atomserve_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec

    d, eps, hd = cfg["hidden_size"], cfg["rms_norm_eps"], cfg["head_dim"]
    layers = []
    for i in range(2):
        p = f"model.layers.{i}."
        if kinds == "cuda":
            mixer = PartSpec("gqa_attention", dict(num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
                             head_dim=hd, qk_norm_eps=eps, position=PartSpec("rotary", dict(head_dim=hd, theta=cfg["rope_theta"]))),
                             p + "self_attn.")  # fmt: skip
            ff, norm = PartSpec("swiglu", dict(intermediate_size=cfg["intermediate_size"]), p + "mlp."), "rms_norm"
        else:
            mixer = PartSpec("torch_attention", dict(num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
                             head_dim=hd, eps=eps, theta=cfg["rope_theta"]), p + "self_attn.")  # fmt: skip
            ff, norm = PartSpec("torch_swiglu", dict(intermediate_size=cfg["intermediate_size"]), p + "mlp."), "torch_rms_norm"
        layers.append(LayerSpec("pre_norm", mixer, ff, PartSpec(norm, dict(eps=eps), p + "input_layernorm."),
                                PartSpec(norm, dict(eps=eps), p + "post_attention_layernorm.")))  # fmt: skip
    t = "" if kinds == "cuda" else "torch_"
    return ModelSpec(
        hidden_size=d, vocab_size=cfg["vocab_size"], max_positions=512,
        embedding=PartSpec("token_embedding" if kinds == "cuda" else "torch_embedding", dict(vocab_size=cfg["vocab_size"]), "model.embed_tokens."),
        layers=tuple(layers),
        schedule=(LayerCall(0), LayerCall(1), LayerCall(0), LayerCall(1, cache_from=1)),
        final_norm=PartSpec(t + "rms_norm", dict(eps=eps), "model.norm."),
        head=PartSpec("lm_head" if kinds == "cuda" else "torch_head", dict(vocab_size=cfg["vocab_size"], tied=False), "lm_head."),
    )  # fmt: skip


def test_a_layer_called_twice_and_a_layer_reading_anothers_cache():
    cfg = {**TINY["b"][0], "num_hidden_layers": 2}
    w = checkpoint(cfg, seed=12)
    ids = prompts(cfg, [37], seed=1)[0]
    cuts = [5, 2, 13, 1, 1, 15]
    ref_whole, ref_cut = run_whole_and_cut(custom_model(shared_cache_spec(cfg, "torch"), w, "cpu", torch.float32), 8, ids, cuts, "cpu")
    assert rel_error(ref_cut, ref_whole) < 1e-5
    model = custom_model(shared_cache_spec(cfg, "cuda"), w, "cuda", torch.float32)
    assert [kv is not None for kv, _ in model.cache_requirements()] == [True, True, True, False]
    whole, cut = run_whole_and_cut(model, 8, ids, cuts, "cuda")
    assert rel_error(whole, ref_whole) < FLOAT32_TOLERANCE and rel_error(cut, ref_whole) < FLOAT32_TOLERANCE
    # and it differs from the plain four-layer stack, i.e. the order really was followed
    assert rel_error(whole, plain.forward(w, cfg, ids)) > 1e-3


def test_a_toy_mixer_with_state_of_its_own_is_registered_built_and_stepped():
    """Layer 0 is the package's attention, layer 1 the test's EMA mixer (state in the request's
    slot). Cut into portions and mixed with another request, it gives what it gives whole, and
    the mixer matches its own recurrence."""
    from atomserve_b200.cache import CacheManager
    from atomserve_b200.engine.runner import ModelRunner, Row
    from atomserve_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec, build_model

    cfg = {**TINY["a"][0], "num_hidden_layers": 2}
    d, eps, hd = cfg["hidden_size"], cfg["rms_norm_eps"], cfg["head_dim"]
    w = checkpoint(cfg, seed=13)
    g = torch.Generator().manual_seed(2)
    w["model.layers.1.ema.in_proj.weight"] = (torch.randn(d, d, generator=g) * 0.05).bfloat16().float()
    attn = PartSpec("gqa_attention", dict(num_heads=4, num_kv_heads=2, head_dim=hd, qk_norm_eps=eps,
                    position=PartSpec("rotary", dict(head_dim=hd, theta=cfg["rope_theta"]))), "model.layers.0.self_attn.")  # fmt: skip
    layers = []
    for i, mixer in enumerate([attn, PartSpec("ema_mixer", dict(decay=0.8), "model.layers.1.ema.")]):
        p = f"model.layers.{i}."
        layers.append(LayerSpec("pre_norm", mixer, PartSpec("swiglu", dict(intermediate_size=cfg["intermediate_size"]), p + "mlp."),
                                PartSpec("rms_norm", dict(eps=eps), p + "input_layernorm."),
                                PartSpec("rms_norm", dict(eps=eps), p + "post_attention_layernorm.")))  # fmt: skip
    spec = ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], max_positions=512,
                     embedding=PartSpec("token_embedding", dict(vocab_size=cfg["vocab_size"]), "model.embed_tokens."),
                     layers=tuple(layers), schedule=(LayerCall(0), LayerCall(1)),
                     final_norm=PartSpec("rms_norm", dict(eps=eps), "model.norm."),
                     head=PartSpec("lm_head", dict(vocab_size=cfg["vocab_size"], tied=True), "lm_head."))  # fmt: skip
    model = build_model(spec)
    wanted = {s.name for s in model.tensor_specs()}
    model.load({k: v.cuda() for k, v in w.items() if k in wanted})
    assert model.cache_requirements()[1][0] is None and model.cache_requirements()[1][1][0].name == "ema"

    a, b = prompts(cfg, [30, 12], seed=3)
    whole = {}
    for name, ids in (("a", a), ("b", b)):
        cache = CacheManager(model.cache_requirements(), 16, 16, 4, torch.float32, "cuda")
        runner = ModelRunner(model, cache)
        assert not runner.use_graphs  # state updated in place: stepped eagerly
        rc = cache.new_request()
        cache.admit(rc), cache.reserve(rc, 0, len(ids))
        whole[name] = runner.step([Row(ids, 0, rc, list(range(len(ids))))]).cpu()
    cache = CacheManager(model.cache_requirements(), 16, 16, 4, torch.float32, "cuda")
    runner = ModelRunner(model, cache)
    ra, rb = cache.new_request(), cache.new_request()
    cache.admit(ra), cache.admit(rb)
    got_a, got_b, at_a, at_b = [], [], 0, 0
    for na, nb in ((7, 0), (2, 5), (1, 1), (11, 1), (1, 5), (8, 0)):
        rows = []
        if na:
            cache.reserve(ra, at_a, na)
            rows.append(Row(a[at_a : at_a + na], at_a, ra, list(range(na))))
        if nb:
            cache.reserve(rb, at_b, nb)
            rows.append(Row(b[at_b : at_b + nb], at_b, rb, list(range(nb))))
        out = runner.step(rows).cpu()
        got_a.append(out[:na]), got_b.append(out[na:])
        at_a, at_b = at_a + na, at_b + nb
    assert rel_error(torch.cat(got_a), whole["a"]) < FLOAT32_TOLERANCE
    assert rel_error(torch.cat(got_b), whole["b"]) < FLOAT32_TOLERANCE
    # a slot handed to a new request starts from zero state
    cache.free(rb)
    rc = cache.new_request()
    cache.admit(rc), cache.reserve(rc, 0, len(b))
    again = runner.step([Row(b, 0, rc, list(range(len(b))))]).cpu()
    assert rel_error(again, whole["b"]) < FLOAT32_TOLERANCE
    # the mixer alone against its recurrence
    mixer = model.blocks[1].mixer
    h = torch.randn(9, d, generator=g).cuda()
    view = cache.entry_view(1)
    slot = cache.state.take()
    y = mixer.forward(h, torch.zeros_like(h), step_context([9], [0], [slot]), view).cpu()
    assert torch.allclose(y, toy_parts.ema_reference((h @ mixer.w.T).cpu(), 0.8), atol=1e-5)


def routed_spec(cfg, kinds):
    """Two layers: the first with the dense feed-forward, the second with the test's routed one."""
    from atomserve_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec

    d, eps, hd = cfg["hidden_size"], cfg["rms_norm_eps"], cfg["head_dim"]
    t = "" if kinds == "cuda" else "torch_"
    layers = []
    for i in range(2):
        p = f"model.layers.{i}."
        if kinds == "cuda":
            mixer = PartSpec("gqa_attention", dict(num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
                             head_dim=hd, qk_norm_eps=eps, position=PartSpec("rotary", dict(head_dim=hd, theta=cfg["rope_theta"]))),
                             p + "self_attn.")  # fmt: skip
        else:
            mixer = PartSpec("torch_attention", dict(num_heads=cfg["num_attention_heads"], num_kv_heads=cfg["num_key_value_heads"],
                             head_dim=hd, eps=eps, theta=cfg["rope_theta"], window=None), p + "self_attn.")  # fmt: skip
        dense = PartSpec(t + "swiglu", dict(intermediate_size=cfg["intermediate_size"]), p + "mlp.")
        routed = PartSpec("toy_top1_experts", dict(num_experts=3, expert_size=40), p + "moe.")
        layers.append(LayerSpec("pre_norm", mixer, routed if i else dense,
                                PartSpec(t + "rms_norm", dict(eps=eps), p + "input_layernorm."),
                                PartSpec(t + "rms_norm", dict(eps=eps), p + "post_attention_layernorm.")))  # fmt: skip
    return ModelSpec(
        hidden_size=d, vocab_size=cfg["vocab_size"], max_positions=512,
        embedding=PartSpec("token_embedding" if kinds == "cuda" else "torch_embedding", dict(vocab_size=cfg["vocab_size"]), "model.embed_tokens."),
        layers=tuple(layers), schedule=(LayerCall(0), LayerCall(1)),
        final_norm=PartSpec(t + "rms_norm", dict(eps=eps), "model.norm."),
        head=PartSpec("lm_head" if kinds == "cuda" else "torch_head", dict(vocab_size=cfg["vocab_size"], tied=False), "lm_head."),
    )  # fmt: skip


def test_a_toy_feed_forward_with_routing_is_registered_built_and_stepped():
    """The second layer's feed-forward is the test's top-1 router over three small experts. The
    model with the package's CUDA parts around it gives, whole and cut into portions, what the
    same model of torch parts gives on the CPU; and the routed part alone matches a token-by-token
    restatement that really does send tokens to different experts."""
    cfg = {**TINY["b"][0], "num_hidden_layers": 2}
    d = cfg["hidden_size"]
    w = checkpoint(cfg, seed=21)
    g = torch.Generator().manual_seed(5)
    for k in [k for k in w if k.startswith("model.layers.1.mlp.")]:
        del w[k]
    w["model.layers.1.moe.router.weight"] = (torch.randn(3, d, generator=g) * 0.5).bfloat16().float()
    for x in range(3):
        for n, shape in (("gate", (40, d)), ("up", (40, d)), ("down", (d, 40))):
            w[f"model.layers.1.moe.experts.{x}.{n}_proj.weight"] = (torch.randn(shape, generator=g) * 0.1).bfloat16().float()
    ids = prompts(cfg, [41], seed=2)[0]
    cuts = [9, 2, 17, 1, 1, 11]
    ref_whole, ref_cut = run_whole_and_cut(custom_model(routed_spec(cfg, "torch"), w, "cpu", torch.float32), 8, ids, cuts, "cpu")
    assert rel_error(ref_cut, ref_whole) < 1e-5
    model = custom_model(routed_spec(cfg, "cuda"), w, "cuda", torch.float32)
    whole, cut = run_whole_and_cut(model, 8, ids, cuts, "cuda")
    assert rel_error(whole, ref_whole) < FLOAT32_TOLERANCE and rel_error(cut, ref_whole) < FLOAT32_TOLERANCE

    ff = model.blocks[1].feed_forward
    h = torch.randn(24, d, generator=g)
    got = ff.forward(h.cuda(), torch.zeros(24, d, device="cuda"), None).cpu()
    logits = h @ w["model.layers.1.moe.router.weight"].T
    chosen = logits.argmax(-1)
    assert len(set(chosen.tolist())) >= 2
    for t in range(24):
        x = int(chosen[t])
        gate, up, down = (w[f"model.layers.1.moe.experts.{x}.{n}_proj.weight"] for n in ("gate", "up", "down"))
        y = (torch.nn.functional.silu(h[t] @ gate.T) * (h[t] @ up.T)) @ down.T * torch.softmax(logits[t], -1)[x]
        assert torch.allclose(got[t], y, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_another_position_encoding_through_the_attention_part(dtype):
    """The package's attention with the test's position encoding (positions compressed by 4, 32
    of 48 head elements rotated) and no q/k norm: two portions through its cache equal causal
    grouped-query attention written out here in float64."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, H, KV, hd, bs, T, theta, factor, rd = 56, 4, 2, 48, 4, 21, 5e3, 4.0, 32
    g = torch.Generator().manual_seed(7)
    names = {"q_proj": (H * hd, d), "k_proj": (KV * hd, d), "v_proj": (KV * hd, d), "o_proj": (d, H * hd)}
    w = {n: (torch.randn(s, generator=g) * 0.1).bfloat16().float() for n, s in names.items()}
    part = build_part("mixer", PartSpec("gqa_attention", dict(
        num_heads=H, num_kv_heads=KV, head_dim=hd, qk_norm_eps=None,
        position=PartSpec("toy_interpolated_rotary", dict(head_dim=hd, theta=theta, factor=factor, rotary_dim=rd))), "a."), d)  # fmt: skip
    part.load({f"a.{n}.weight": v.cuda().to(dtype) for n, v in w.items()})
    h = torch.randn(T, d, generator=g).bfloat16().float()
    res = torch.randn(T, d, generator=g).bfloat16().float()

    pos = torch.arange(T)
    q = toy_parts.interpolated_rotary_reference((h @ w["q_proj"].T).view(T, H, hd), pos, theta, factor, rd)
    k = toy_parts.interpolated_rotary_reference((h @ w["k_proj"].T).view(T, KV, hd), pos, theta, factor, rd)
    v = (h @ w["v_proj"].T).view(T, KV, hd).double()
    k, v = k.repeat_interleave(H // KV, dim=1), v.repeat_interleave(H // KV, dim=1)
    scores = torch.einsum("thd,shd->hts", q, k) * hd**-0.5
    scores = scores.masked_fill(pos[None, :, None] < pos[None, None, :], float("-inf"))
    attn = torch.einsum("hts,shd->thd", torch.softmax(scores, -1), v).reshape(T, H * hd)
    ref = (res.double() + attn @ w["o_proj"].double().T).float()

    view = CacheView(k=torch.zeros(8, KV, bs, hd, device="cuda", dtype=dtype), block_size=bs)
    view.v = torch.zeros_like(view.k)
    table = [4, 1, 6, 0, 3, 7]
    view.block_tables = torch.tensor([table], dtype=torch.int32, device="cuda")
    outs = []
    for start, n in ((0, 13), (13, 8)):
        view.slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(start, start + n)], dtype=torch.int32, device="cuda")
        outs.append(part.forward(h[start : start + n].cuda().to(dtype), res[start : start + n].cuda().to(dtype),
                                 step_context([n], [start]), view))  # fmt: skip
    got = torch.cat(outs).float().cpu()
    assert rel_error(got, ref) < (1e-5 if dtype == torch.float32 else 2e-2)
    # and the encoding matters: the package's own rotary at the same theta gives something else
    own = build_part("mixer", PartSpec("gqa_attention", dict(
        num_heads=H, num_kv_heads=KV, head_dim=hd, qk_norm_eps=None,
        position=PartSpec("rotary", dict(head_dim=hd, theta=theta))), "a."), d)  # fmt: skip
    own.load({f"a.{n}.weight": v.cuda().to(dtype) for n, v in w.items()})
    view.slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(T)], dtype=torch.int32, device="cuda")
    other = own.forward(h.cuda().to(dtype), res.cuda().to(dtype), step_context([T], [0]), view).float().cpu()
    assert rel_error(other, ref) > 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_position_encoding_that_is_no_rotation_by_frequency(dtype):
    """The package's attention with an encoding that has no fused form (angle = sqrt(position) x
    frequency): the part normalises q and k, lets the encoding's own `encode` work the positions
    in, then stores. Two portions through its cache equal the longhand in float64."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, H, KV, hd, bs, T, theta, eps = 64, 4, 2, 32, 4, 21, 2e3, 1e-5
    g = torch.Generator().manual_seed(9)
    names = {"q_proj": (H * hd, d), "k_proj": (KV * hd, d), "v_proj": (KV * hd, d), "o_proj": (d, H * hd)}
    w = {n: (torch.randn(s, generator=g) * 0.1).bfloat16().float() for n, s in names.items()}
    gains = {n: 1 + 0.1 * torch.randn(hd, generator=g) for n in ("q_norm", "k_norm")}
    part = build_part("mixer", PartSpec("gqa_attention", dict(
        num_heads=H, num_kv_heads=KV, head_dim=hd, qk_norm_eps=eps,
        position=PartSpec("toy_sqrt_rotation", dict(head_dim=hd, theta=theta))), "a."), d)  # fmt: skip
    assert part.position.fused_rotary() is None
    part.load({**{f"a.{n}.weight": v.cuda().to(dtype) for n, v in w.items()},
               **{f"a.{n}.weight": v.cuda() for n, v in gains.items()}})  # fmt: skip
    h = torch.randn(T, d, generator=g).bfloat16().float()
    res = torch.randn(T, d, generator=g).bfloat16().float()

    pos = torch.arange(T)
    q = plain.rms_norm((h @ w["q_proj"].T).view(T, H, hd).double(), gains["q_norm"].double(), eps)
    k = plain.rms_norm((h @ w["k_proj"].T).view(T, KV, hd).double(), gains["k_norm"].double(), eps)
    q, k = toy_parts.sqrt_rotation_reference(q, pos, theta), toy_parts.sqrt_rotation_reference(k, pos, theta)
    v = (h @ w["v_proj"].T).view(T, KV, hd).double()
    ref = (res.double() + plain.attention(q, k, v).reshape(T, H * hd) @ w["o_proj"].double().T).float()

    view = CacheView(k=torch.zeros(8, KV, bs, hd, device="cuda", dtype=dtype), block_size=bs)
    view.v = torch.zeros_like(view.k)
    table = [4, 1, 6, 0, 3, 7]
    view.block_tables = torch.tensor([table], dtype=torch.int32, device="cuda")
    outs = []
    for start, n in ((0, 13), (13, 8)):
        view.slots = torch.tensor([table[p // bs] * bs + p % bs for p in range(start, start + n)], dtype=torch.int32, device="cuda")
        outs.append(part.forward(h[start : start + n].cuda().to(dtype), res[start : start + n].cuda().to(dtype),
                                 step_context([n], [start]), view))  # fmt: skip
    got = torch.cat(outs).float().cpu()
    assert rel_error(got, ref) < (1e-5 if dtype == torch.float32 else 2e-2)
    # the rule matters: with plain positions instead of their square roots the result differs
    q2 = plain.apply_rope(q.float(), plain.rope_angles(pos, hd, theta))
    assert (q2.double() - q).abs().max() > 1e-2


def test_a_toy_mixer_whose_pages_hold_one_tensor_runs_beside_the_packages_attention():
    """Layer 0 is the package's attention (pages of keys and values), layer 1 the test's latent
    mixer (pages of one narrow tensor): two cache groups of different page contents in one model,
    stepped by the package's runner on the GPU, whole and cut into portions, mixed with a second
    request; the result is the CPU model's of torch parts."""
    from atomserve_b200.cache import CacheManager
    from atomserve_b200.parts import LayerCall, LayerSpec, ModelSpec, PartSpec

    cfg = {**TINY["a"][0], "num_hidden_layers": 2}
    d, eps, hd, rank, bs = cfg["hidden_size"], cfg["rms_norm_eps"], cfg["head_dim"], 12, 16
    w = checkpoint(cfg, seed=14)
    g = torch.Generator().manual_seed(4)
    for k in [k for k in w if k.startswith("model.layers.1.self_attn.")]:
        del w[k]
    for n, shape in (("down", (rank, d)), ("query", (rank, d)), ("up", (d, rank))):
        w[f"model.layers.1.latent.{n}.weight"] = (torch.randn(shape, generator=g) * 0.3).bfloat16().float()

    def spec(kinds):
        t = "" if kinds == "cuda" else "torch_"
        if kinds == "cuda":
            attn = PartSpec("gqa_attention", dict(num_heads=4, num_kv_heads=2, head_dim=hd, qk_norm_eps=eps,
                            position=PartSpec("rotary", dict(head_dim=hd, theta=cfg["rope_theta"]))), "model.layers.0.self_attn.")  # fmt: skip
        else:
            attn = PartSpec("torch_attention", dict(num_heads=4, num_kv_heads=2, head_dim=hd, eps=eps, theta=cfg["rope_theta"]),
                            "model.layers.0.self_attn.")  # fmt: skip
        layers = []
        for i, mixer in enumerate([attn, PartSpec("latent_mixer", dict(rank=rank), "model.layers.1.latent.")]):
            p = f"model.layers.{i}."
            layers.append(LayerSpec("pre_norm", mixer, PartSpec(t + "swiglu", dict(intermediate_size=cfg["intermediate_size"]), p + "mlp."),
                                    PartSpec(t + "rms_norm", dict(eps=eps), p + "input_layernorm."),
                                    PartSpec(t + "rms_norm", dict(eps=eps), p + "post_attention_layernorm.")))  # fmt: skip
        return ModelSpec(hidden_size=d, vocab_size=cfg["vocab_size"], max_positions=512,
                         embedding=PartSpec("token_embedding" if kinds == "cuda" else "torch_embedding", dict(vocab_size=cfg["vocab_size"]), "model.embed_tokens."),
                         layers=tuple(layers), schedule=(LayerCall(0), LayerCall(1)),
                         final_norm=PartSpec(t + "rms_norm", dict(eps=eps), "model.norm."),
                         head=PartSpec("lm_head" if kinds == "cuda" else "torch_head", dict(vocab_size=cfg["vocab_size"], tied=True), "lm_head."))  # fmt: skip

    ids = prompts(cfg, [37], seed=2)[0]
    cuts = [5, 2, 13, 1, 1, 15]
    ref_whole, ref_cut = run_whole_and_cut(custom_model(spec("torch"), w, "cpu", torch.float32), bs, ids, cuts, "cpu")
    assert rel_error(ref_cut, ref_whole) < 1e-5
    model = custom_model(spec("cuda"), w, "cuda", torch.float32)
    cache = CacheManager(model.cache_requirements(), bs, 8, 2, torch.float32, "cuda")
    assert [sorted(g.pools) for g in cache.groups] == [["k", "v"], ["latent"]]
    whole, cut = run_whole_and_cut(model, bs, ids, cuts, "cuda")
    assert rel_error(whole, ref_whole) < FLOAT32_TOLERANCE and rel_error(cut, ref_whole) < FLOAT32_TOLERANCE
