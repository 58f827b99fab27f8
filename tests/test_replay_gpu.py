"""The engine's step function, cache and kernels against the plain implementation, through the
trace replayer: every way of cutting requests into steps must give the oracle's logits."""

import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from helpers import BF16_REPORT, Oracle, check, checkpoint, mixed_trace, prompts, write_folder
from tiny_configs import TINY

pytestmark = pytest.mark.gpu
DTYPES = ["float32", "bfloat16"]
LENGTHS = {"a": [5, 17, 33, 70], "b": [1, 9, 24, 40, 75], "c": [3, 50, 90, 41], "d": [45, 200, 9, 330],
           "e": [41, 150, 12, 230]}  # fmt: skip


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, block size, folder, prompts, oracle per prompt). An oracle is the
    float32 logits with their bfloat16 allowance attached (`Oracle`)."""
    out = {}
    for name, (cfg, bs) in TINY.items():
        w = checkpoint(cfg, seed=21)
        folder = write_folder(cfg, w, tmp_path_factory.mktemp(f"tiny_{name}"))
        ps = prompts(cfg, LENGTHS[name], seed=4)
        out[name] = (cfg, bs, folder, ps, [Oracle(w, cfg, p) for p in ps])
    return out


def replayer(folder, dtype, bs, max_tokens, graphs=True, **more):
    from atomserve_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, bs, cuda_graphs=graphs, **more)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_each_request_alone_and_whole(models, name, dtype):
    cfg, bs, folder, ps, oracle = models[name]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    for i, (p, ref) in enumerate(zip(ps, oracle)):
        logits = rp.step([dict(id=i, tokens=p, want=list(range(len(p))))], end=[i])
        check(logits, ref, dtype, f"{name} request {i} whole")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_prefill_then_last_32_one_by_one(models, name, dtype):
    cfg, bs, folder, ps, oracle = models[name]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    for i, (p, ref) in enumerate(zip(ps, oracle)):
        head = max(len(p) - 32, 0)
        got = []
        if head:
            got.append(rp.step([dict(id=i, tokens=p[:head], want=[head - 1])], end=[]))
            check(got[0], ref[head - 1 : head], dtype, f"{name} request {i} head")
        for j in range(head, len(p)):
            logits = rp.step([dict(id=i, tokens=[p[j]], want=[0])], end=[i] if j == len(p) - 1 else [])
            check(logits, ref[j : j + 1], dtype, f"{name} request {i} position {j}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_portions_of_changing_size(models, name, dtype):
    cfg, bs, folder, ps, oracle = models[name]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    sizes = [2, 7, 3, 16, 2, 17, 5, 31, 2, 9]
    for i, (p, ref) in enumerate(zip(ps, oracle)):
        at, k = 0, i
        while at < len(p):
            n = min(sizes[k % len(sizes)], len(p) - at)
            k += 1
            last = at + n == len(p)
            logits = rp.step([dict(id=i, tokens=p[at : at + n], want=list(range(n)))], end=[i] if last else [])
            check(logits, ref[at : at + n], dtype, f"{name} request {i} portion {at}:{at + n}")
            at += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["a", "b", "c", "d", "e"])
def test_mixed_requests_reusing_pages(models, name, dtype):
    """Up to four live requests, portions beside single tokens, in a pool so small that pages
    freed by finished requests are taken again by later ones; every request appears three times,
    so that later copies run entirely on used pages."""
    cfg, bs, folder, ps, oracle = models[name]
    ps2, oracle2 = ps * 3, oracle * 3
    biggest = sorted((-(-len(p) // 64) * 64 for p in ps), reverse=True)
    rp = replayer(folder, dtype, bs, sum(biggest[:4]))
    rng = np.random.default_rng(7)
    for entries, end in mixed_trace(ps2, rng):
        logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            check(logits[row : row + n], oracle2[e["id"]][e["at"] : e["at"] + n], dtype,
                  f"{name} request {e['id']} at {e['at']}")  # fmt: skip
            row += n
    total_tokens = sum(len(p) for p in ps2)
    assert total_tokens > rp.cache.num_blocks * bs, "the pool was large enough to never reuse a page"


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding(models, dtype):
    """300 tokens one by one (across many pages and, for config c, far beyond its window)."""
    for name in ("b", "c", "d", "e"):
        cfg, bs, folder, _, _ = models[name]
        w = checkpoint(cfg, seed=21)
        p = prompts(cfg, [300], seed=9)[0]
        ref = Oracle(w, cfg, p)
        for graphs in (True, False):
            rp = replayer(folder, dtype, bs, 320, graphs)
            for j, t in enumerate(p):
                logits = rp.step([dict(id="x", tokens=[t], want=[0])], end=[])
                if j % 7 == 0 or j > 290:
                    check(logits, ref[j : j + 1], dtype, f"{name} decode position {j} graphs={graphs}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,live", [("a", 70), ("d", 150)])
def test_many_requests_decode_together(models, name, live, dtype):
    """70 and 150 live requests of different lengths: their prompts in a few mixed steps, then
    single tokens of all of them in one step each (the batch sizes where the GEMM runs its
    medium-token shapes and the decode graphs their large buckets)."""
    cfg, bs, folder, _, _ = models[name]
    w = checkpoint(cfg, seed=21)
    lengths = [3 + (7 * i) % 23 for i in range(live)]
    ps = prompts(cfg, [n + 3 for n in lengths], seed=11)  # three more tokens each, fed one by one
    rp = replayer(folder, dtype, bs, live * 64, max_live=live)
    for first in range(0, live, 40):  # prompts, forty requests a step
        ids = range(first, min(first + 40, live))
        rp.step([dict(id=str(i), tokens=ps[i][: lengths[i]], want=[]) for i in ids], end=[])
    refs = {i: Oracle(w, cfg, ps[i]) for i in range(0, live, 13)}  # a sample of the requests is checked
    for k in range(3):
        logits = rp.step([dict(id=str(i), tokens=[ps[i][lengths[i] + k]], want=[0]) for i in range(live)], end=[])
        assert logits.shape[0] == live
        for i, ref in refs.items():
            at = lengths[i] + k
            check(logits[i : i + 1], ref[at : at + 1], dtype, f"{name} {live} live, request {i} position {at}")


LONG = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=300, hidden_size=128, intermediate_size=320,
    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=1, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=True,
    max_position_embeddings=16384, hidden_act="silu",
)  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
def test_decoding_across_the_graph_context_buckets(tmp_path, dtype):
    """One request of 8,210 tokens: decoded token by token from 2,040 to 2,060 and from 8,185 to
    the end, which takes the decode graphs over the context buckets at 2,048 (then 2,560) and at
    8,192 (then 9,216), each with another plan of key partitions; between them a portion of
    6,125 tokens behind 2,060 cached ones. Every wanted row against the plain implementation."""
    w = checkpoint(LONG, seed=5)
    folder = write_folder(LONG, w, tmp_path / "long")
    p = prompts(LONG, [8210], seed=1)[0]
    ref = Oracle(w, LONG, p)
    rp = replayer(folder, dtype, 16, 8256)
    assert rp.runner.use_graphs

    def run(at, n, want):
        logits = rp.step([dict(id="x", tokens=p[at : at + n], want=want)], end=[])
        check(logits, ref[[at + j for j in want]], dtype, f"long request, {n} tokens at {at}")

    run(0, 2040, [0, 1000, 2039])
    for at in range(2040, 2060):
        run(at, 1, [0])
    run(2060, 6125, [0, 5, 3000, 6124])
    for at in range(8185, 8210):
        run(at, 1, [0])
    buckets = sorted({key[-1] for key in rp.runner._graphs._entries})
    assert buckets == [2048, 2560, 8192, 9216], buckets


def test_window_pages_are_given_back(models):
    cfg, bs, folder, _, _ = models["c"]
    rp = replayer(folder, "float32", bs, 320)
    p = prompts(cfg, [200], seed=2)[0]
    for t in p:
        rp.step([dict(id="w", tokens=[t], want=[])], end=[])
    rc, _ = rp.live["w"]
    full = [g for g in rp.cache.groups if g.window is None][0]
    windowed = [g for g in rp.cache.groups if g.window is not None][0]
    held = {id(g): sum(b >= 0 for b in t) for g, t in zip(rp.cache.groups, rc.block_tables)}
    assert held[id(full)] == -(-200 // bs)
    assert held[id(windowed)] <= -(-cfg["sliding_window"] // bs) + 1
    assert windowed.allocator.num_free == rp.cache.num_blocks - held[id(windowed)]


def test_trace_run_program(models, tmp_path):
    """The program itself: steps on stdin, `done` lines, .f32 files, exit code 0."""
    cfg, bs, folder, ps, oracle = models["b"]
    steps = [
        dict(step=0, entries=[dict(id="a", tokens=ps[2][:10], want=[0, 9]), dict(id="b", tokens=ps[1], want=[8])], end=["b"]),
        dict(step=1, entries=[dict(id="a", tokens=ps[2][10:12], want=[])], end=[]),
        dict(step=2, entries=[dict(id="a", tokens=ps[2][12:], want=[len(ps[2]) - 13])], end=["a"]),
    ]
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    for dtype in DTYPES:
        out = tmp_path / dtype
        done = subprocess.run(
            [sys.executable, str(root / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
             "--out", str(out), "--max-tokens", "128", "--block-size", str(bs)],
            input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=600,
        )  # fmt: skip
        assert done.returncode == 0, done.stderr[-2000:]
        assert done.stdout.split() == ["done", "0", "done", "1", "done", "2"]
        assert not (out / "1.f32").exists()
        s0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(3, cfg["vocab_size"]))
        check(s0[:2], oracle[2][[0, 9]], dtype, "step 0 request a")
        check(s0[2:], oracle[1][8:9], dtype, "step 0 request b")
        s2 = torch.from_numpy(np.fromfile(out / "2.f32", dtype="<f4").reshape(1, cfg["vocab_size"]))
        check(s2, oracle[2][-1:], dtype, "step 2")


def test_zz_report_bfloat16_margins():
    """Not a check: prints how much of its allowance the bfloat16 engine used."""
    if BF16_REPORT:
        worst = sorted(BF16_REPORT, key=lambda x: -x[1])[:5]
        mean = sum(r for _, r in BF16_REPORT) / len(BF16_REPORT)
        print(f"\nbfloat16 error / allowance: mean {mean:.2f} over {len(BF16_REPORT)} checks; worst {worst}")
