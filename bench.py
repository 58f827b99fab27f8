"""Decode and prefill throughput of the engine at Qwen3-8B sizes on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--impl reference]

A step is one decode step. The default run builds a random-weight model with the layer sizes of
Qwen3-8B, prefills 8 requests of 2,048 synthetic token ids and times K decode steps on the
device (CUDA events); the same through the engine's public API with host tokens in and out
gives `e2e`. It also times a 2,048-token prefill and decode at batch 1 and 64, and prints one
JSON line. Weights (15 GB) are read once per step and exceed the L2 cache, so no flush is
needed between timed iterations.
"""

from __future__ import annotations

import argparse
import dataclasses
import json
import pathlib
import subprocess
import sys
import tempfile
import time

ROOT = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

QWEN3_8B = dict(
    architectures=["Qwen3ForCausalLM"], vocab_size=151936, hidden_size=4096, intermediate_size=12288,
    num_hidden_layers=36, num_attention_heads=32, num_key_value_heads=8, head_dim=128,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=40960,
)  # fmt: skip
# the other two shapes that the reference's benchmark list names (its bench/engine.py runs whatever
# checkpoint it is given); `--shape` picks one for the --only runs
QWEN3_14B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 17408, "num_hidden_layers": 40, "num_attention_heads": 40}
QWEN3_32B = {**QWEN3_8B, "hidden_size": 5120, "intermediate_size": 25600, "num_hidden_layers": 64, "num_attention_heads": 64}
SHAPES = {"8b": QWEN3_8B, "14b": QWEN3_14B, "32b": QWEN3_32B}
PROMPT_TOKENS = 2048
CONTEXT = 4096
BLOCK_SIZE = 16
PUBLISHED_8B_BATCH1 = 15.7  # tok/s, the reference's Qwen3-8B bf16 batch-1 decode on an M4 Pro


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        raw = json.loads(path.read_text())
        return {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                "bf16_tflops_sustained": float(raw.get("bf16_tflops_sustained", raw["bf16_tflops"])), "source": "measured"}  # fmt: skip
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def prompts(batch: int, length: int) -> list[list[int]]:
    """Distinct synthetic prompts (the reference's bench/engine.py:90-92)."""
    return [[(1000 + 37 * b + i) % 150000 for i in range(length)] for b in range(batch)]


class ClockSampler:
    """nvidia-smi's clocks and throttle reasons, sampled every 100 ms while the block runs."""

    _folder = None

    def __init__(self, name: str = "bench_clocks.csv"):
        if ClockSampler._folder is None:
            ClockSampler._folder = tempfile.TemporaryDirectory(prefix="atomserve_b200_bench_")
        self.proc, self.path = None, pathlib.Path(ClockSampler._folder.name) / name

    def __enter__(self):
        try:
            self.file = open(self.path, "w")
            self.proc = subprocess.Popen(
                ["nvidia-smi", "--query-gpu=clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                 "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                 "clocks_event_reasons.sw_power_cap", "--format=csv,noheader,nounits", "-lms", "100", "-i", "0"],
                stdout=self.file, stderr=subprocess.DEVNULL,
            )  # fmt: skip
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            self.proc.wait()
            self.file.close()

    def summary(self) -> dict:
        rows = []
        try:
            for line in self.path.read_text().splitlines():
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 7 and parts[0].isdigit():
                    rows.append(parts)
        except OSError:
            pass
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(r[0]) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(rows[0][1]), "reasons": reasons, "samples": len(rows)}


def build_engine(layers: int, max_seqs: int, shape: dict = QWEN3_8B, context: int = CONTEXT, budget: int = PROMPT_TOKENS):
    import torch

    from atomserve_b200.config import EngineConfig
    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.weights import random_model

    _, config = config_from_dict({**shape, "num_hidden_layers": layers})
    model = random_model(config, seed=0, dtype="bfloat16", device="cuda")
    blocks = max_seqs * (context // BLOCK_SIZE) + 64
    engine_config = EngineConfig(block_size=BLOCK_SIZE, num_blocks=blocks, max_num_seqs=max_seqs,
                                 max_num_batched_tokens=budget, max_model_len=context,
                                 enable_prefix_caching=False)  # fmt: skip
    torch.cuda.synchronize()
    return config, model, create_engine(model, engine_config, sampler_seed=0)


def step_bytes(config, batch: int, context: int) -> float:
    """Bytes a decode step has to read: every weight it uses once (all layers and the head;
    embedding rows are negligible) and the cached keys and values of the live requests."""
    c = config
    per_layer = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * c.hidden_size \
        + c.hidden_size * c.num_attention_heads * c.head_dim + 3 * c.intermediate_size * c.hidden_size
    weights = 2 * (c.num_hidden_layers * per_layer + c.vocab_size * c.hidden_size)
    kv = 2 * 2 * c.num_key_value_heads * c.head_dim * c.num_hidden_layers * context * batch
    return float(weights + kv)


def prefill_flops(config, tokens: int) -> float:
    c = config
    per_layer = (c.num_attention_heads + 2 * c.num_key_value_heads) * c.head_dim * c.hidden_size \
        + c.hidden_size * c.num_attention_heads * c.head_dim + 3 * c.intermediate_size * c.hidden_size
    linear = 2.0 * tokens * c.num_hidden_layers * per_layer + 2.0 * c.vocab_size * c.hidden_size
    attention = c.num_hidden_layers * 4.0 * c.num_attention_heads * c.head_dim * tokens * tokens / 2
    return linear + attention


def time_decode(engine, batch: int, steps: int, warmup: int, prompt_tokens: int = PROMPT_TOKENS):
    """Prefill `batch` requests (untimed), then time `steps` decode steps two ways: on the
    device around the step function plus argmax, and end to end through Engine.step()."""
    PROMPT_TOKENS = prompt_tokens
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.engine.runner import Row
    from atomserve_b200.engine.sequence import SamplingParams
    from atomserve_b200.ops.library import launches as kernel_launches

    runner, cache = engine.runner, engine.runner.cache
    # --- device-timed: the step function on fixed token ids, positions advancing ---
    reqs = []
    for p in prompts(batch, PROMPT_TOKENS):
        rc = cache.new_request()
        assert cache.admit(rc) and cache.reserve(rc, 0, PROMPT_TOKENS)
        runner.step([Row(p, 0, rc, [])])
        reqs.append(rc)
    pos = PROMPT_TOKENS

    def one_step(position):
        rows = []
        for i, rc in enumerate(reqs):
            assert cache.reserve(rc, position, 1)
            rows.append(Row([(7 + 13 * i + position) % 150000], position, rc, [0]))
        return ops.argmax_rows(runner.step(rows))

    for _ in range(warmup):
        one_step(pos)
        pos += 1
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches_before = kernel_launches()
    start.record()
    for _ in range(steps):
        one_step(pos)
        pos += 1
    end.record()
    torch.cuda.synchronize()
    device_ms = start.elapsed_time(end) / steps
    launches = kernel_launches() - launches_before
    mid_context = PROMPT_TOKENS + warmup + steps // 2
    for rc in reqs:
        cache.free(rc)

    e2e, upload_bytes = time_e2e(engine, batch, steps, warmup, PROMPT_TOKENS)
    return device_ms, launches, mid_context, e2e, upload_bytes


def time_e2e(engine, batch: int, steps: int, warmup: int, prompt_tokens: int, greedy: bool = True):
    """End to end: Engine.step(), host token ids in, sampled ids out, every step; greedy, or the
    reference's default settings (temperature 0.6, top-k 20, top-p 0.95: atomserve/sequence.py:47)."""
    import torch

    from atomserve_b200.engine.sequence import THINKING_PARAMS, SamplingParams

    # long enough that nobody finishes inside the timed region (later requests start later)
    base = SamplingParams(temperature=0.0) if greedy else THINKING_PARAMS
    params = dataclasses.replace(base, max_tokens=warmup + steps + batch + 16, ignore_eos=True)
    handles = [engine.submit(p, params) for p in prompts(batch, prompt_tokens)]
    while any(h.first_token_at is None for h in handles):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    before = engine.num_generated_tokens
    t0 = time.perf_counter()
    for _ in range(steps - 1):
        engine.step()
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    e2e_tokens = engine.num_generated_tokens - before
    upload_bytes = engine.runner.last_upload_bytes  # the packed int32 buffer of a decode step
    while engine.step():
        pass
    for h in handles:
        list(h)
    return e2e_tokens / e2e_s, upload_bytes


def time_prefill_through_engine(model, budget: int, repeats: int, warmup: int) -> float:
    """One cold prompt of 2,048 tokens, one output token, through Engine.generate under a token
    budget per step (512 is the reference's default, atomserve/config.py:75: four portions), as
    the reference times its prefill (bench/engine.py:121-126); milliseconds, CUDA events."""
    import torch

    from atomserve_b200.config import EngineConfig
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.engine.sequence import SamplingParams

    config = EngineConfig(block_size=BLOCK_SIZE, num_blocks=8 * (CONTEXT // BLOCK_SIZE) + 64, max_num_seqs=8,
                          max_num_batched_tokens=budget, max_model_len=CONTEXT, enable_prefix_caching=False)  # fmt: skip
    engine = create_engine(model, config, sampler_seed=0)
    params = SamplingParams(temperature=0.0, max_tokens=1)
    for _ in range(warmup):
        engine.generate(prompts(1, PROMPT_TOKENS), params)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        engine.generate(prompts(1, PROMPT_TOKENS), params)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / repeats


def time_serving(engine, requests: int, decode_tokens: int, seed: int = 0) -> dict:
    """A mixed load through the public API: `requests` prompts of 128 to 2,048 synthetic ids
    submitted at once, `decode_tokens` greedy tokens each; the scheduler cuts the prompts into
    portions under its token budget beside the running decodes. Wall-clock time, host to host."""
    import random

    import torch

    from atomserve_b200.engine.sequence import SamplingParams

    rng = random.Random(seed)
    lengths = [rng.randint(128, 2048) for _ in range(requests)]
    batch = [[(1000 + 37 * b + i) % 150000 for i in range(n)] for b, n in enumerate(lengths)]
    params = SamplingParams(temperature=0.0, max_tokens=decode_tokens, ignore_eos=True)
    engine.generate(batch[:2], SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))  # warm-up: builds, graphs
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    handles = [engine.submit(p, params) for p in batch]
    kinds = {"decode": [0, 0.0], "mixed": [0, 0.0]}  # steps and seconds, by whether a prompt portion was in the step
    last = time.perf_counter()
    while engine.step():  # what Engine.generate does, with a clock read per step (the step ends with a device-to-host read)
        now = time.perf_counter()
        kind = kinds["decode" if engine.last_batch_tokens == engine.last_batch_seqs else "mixed"]
        kind[0] += 1
        kind[1] += now - last
        last = now
    outputs = [list(h) for h in handles]
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    generated = sum(len(o) for o in outputs)
    return {"requests": requests, "prompt_tokens": sum(lengths), "generated_tokens": generated, "seconds": round(seconds, 3),
            "generated_tokens_per_s": round(generated / seconds, 1),
            "total_tokens_per_s": round((generated + sum(lengths)) / seconds, 1),
            "decode_steps": kinds["decode"][0], "decode_step_ms": round(1e3 * kinds["decode"][1] / max(kinds["decode"][0], 1), 3),
            "mixed_steps": kinds["mixed"][0], "mixed_step_ms": round(1e3 * kinds["mixed"][1] / max(kinds["mixed"][0], 1), 3)}  # fmt: skip


def time_prefill(engine, steps: int, warmup: int) -> float:
    import torch

    from atomserve_b200.engine.runner import Row

    runner, cache = engine.runner, engine.runner.cache
    rc = cache.new_request()
    assert cache.admit(rc) and cache.reserve(rc, 0, PROMPT_TOKENS)
    row = [Row(prompts(1, PROMPT_TOKENS)[0], 0, rc, [PROMPT_TOKENS - 1])]
    for _ in range(warmup):
        runner.step(row)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        runner.step(row)
    end.record()
    torch.cuda.synchronize()
    cache.free(rc)
    return start.elapsed_time(end) / steps


def time_gemms(which: str, tokens: list[int], steps: int) -> None:
    """Device time of this package's tcgen05 GEMM and of the vendor library's on the model's
    five weight shapes, replayed from a CUDA graph (no host time), rotating over several weight
    copies so that no call finds its weights in L2. One JSON line per (shape, tokens)."""
    import torch

    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05

    c = QWEN3_8B
    qkv_rows = (c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"]
    shapes = {
        "qkv": (qkv_rows, c["hidden_size"]), "o": (c["hidden_size"], c["num_attention_heads"] * c["head_dim"]),
        "gate_up": (2 * c["intermediate_size"], c["hidden_size"]), "down": (c["hidden_size"], c["intermediate_size"]),
        "lm_head": (c["vocab_size"], c["hidden_size"]),
    }  # fmt: skip

    def graph_time(fn, n):
        for i in range(3):
            fn(i)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for i in range(n):
                fn(i)
        g.replay()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        g.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / n * 1000

    for name, (N, K) in shapes.items():
        if which not in ("all", name):
            continue
        copies = 2 if name == "lm_head" else 6
        ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(copies)]
        for M in tokens:
            if name == "lm_head" and M > 256:
                continue
            x = torch.randn(M, K, device="cuda").bfloat16()
            dt = torch.float32 if name == "lm_head" else torch.bfloat16
            library = graph_time(lambda i: torch.mm(x, ws[i % copies].t(), out_dtype=dt) if dt == torch.float32
                                 else torch.mm(x, ws[i % copies].t()), steps)  # fmt: skip
            mine = graph_time(lambda i: gemm_tcgen05(x, ws[i % copies], None, dt), steps)
            check_gemm_status()
            print(json.dumps({"gemm": name, "tokens": M, "N": N, "K": K, "tcgen05_us": round(mine, 1),
                              "library_us": round(library, 1), "tcgen05_tbs": round(N * K * 2 / mine / 1e6, 2),
                              "tcgen05_tflops": round(2 * M * N * K / mine / 1e6, 1)}))  # fmt: skip
        del ws


def attention_partition_sweep(batches: list[int], contexts: list[int]) -> None:
    """Device time of the decode attention kernel plus its partition merge for every number of key
    partitions, per (batch, context), at the 8B shape's heads; one JSON line each, with the plan
    that the engine's planner picks. CUDA-graph loop, microseconds."""
    import torch

    from atomserve_b200 import ops
    from atomserve_b200.ops.attention import plan_decode_partitions

    c = QWEN3_8B
    H, KV, hd, bs = c["num_attention_heads"], c["num_key_value_heads"], c["head_dim"], BLOCK_SIZE
    for B in batches:
        for ctx in contexts:
            pages = -(-ctx // bs)
            blocks = B * pages + 1
            if blocks * KV * bs * hd * 2 * 2 > 24e9:
                continue
            k = (torch.randn(blocks, KV, bs, hd, device="cuda") * 0.5).bfloat16()
            v = (torch.randn(blocks, KV, bs, hd, device="cuda") * 0.5).bfloat16()
            tables = torch.randperm(blocks - 1, device="cuda")[: B * pages].int().view(B, pages).contiguous()
            q = torch.randn(B, H, hd, device="cuda").bfloat16()
            q_start = torch.arange(B + 1, dtype=torch.int32, device="cuda")
            pos = torch.full((B,), ctx - 1, dtype=torch.int32, device="cuda")
            times = {}
            for want in range(1, 33):
                size = max(256, -(-(-(-ctx // want)) // 64) * 64)
                parts = (ctx - 1) // size + 1
                if parts in times:
                    continue
                plan = (size, parts) if parts > 1 else (1 << 30, 1)

                def run():
                    return ops.paged_attention(q, k, v, tables, q_start, pos, num_requests=B, max_context=ctx, window=None,
                                               scale=hd**-0.5, partitions=plan, host_q_lens=[1] * B)  # fmt: skip

                run()
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph):
                    for _ in range(10):
                        run()
                graph.replay()
                torch.cuda.synchronize()
                start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                start.record()
                graph.replay()
                end.record()
                torch.cuda.synchronize()
                times[parts] = round(start.elapsed_time(end) * 100, 1)
            planned = plan_decode_partitions(B, KV, H // KV, ctx, 0, hd)
            print(json.dumps({"attention": "decode", "batch": B, "context": ctx,
                              "ideal_us": round(B * ctx * KV * hd * 2 * 2 / 7.3e12 * 1e6, 1),
                              "planned_parts": planned[1], "us_by_parts": times}))  # fmt: skip
            del k, v


def time_sampling(batches: list[int], vocab: int) -> None:
    """Device time of the sampling kernels on float32 logits [B, vocab] (normal, standard deviation
    3), from a CUDA-graph loop of 20 calls: greedy, the reference's default settings, top-p alone."""
    import torch

    from atomserve_b200 import ops

    for B in batches:
        logits = torch.randn(B, vocab, device="cuda") * 3
        temperature = torch.full((B,), 0.6, device="cuda")
        top_k = torch.full((B,), 20, dtype=torch.int32, device="cuda")
        no_top_k = torch.zeros(B, dtype=torch.int32, device="cuda")
        top_p = torch.full((B,), 0.95, device="cuda")
        seed = torch.arange(B, dtype=torch.int64, device="cuda")
        counter = torch.zeros(B, dtype=torch.int64, device="cuda")
        cases = {
            "argmax_us": lambda: ops.argmax_rows(logits),
            "top_k20_top_p_us": lambda: ops.sample_rows(logits, temperature, top_k, top_p, seed, counter),
            "top_p_only_us": lambda: ops.sample_rows(logits, temperature, no_top_k, top_p, seed, counter),
        }
        line = {"sampling": "rows", "batch": B, "vocab": vocab}
        for name, fn in cases.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(20):
                    fn()
            graph.replay()
            torch.cuda.synchronize()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            graph.replay()
            end.record()
            torch.cuda.synchronize()
            line[name] = round(start.elapsed_time(end) * 1000 / 20, 1)
        print(json.dumps(line))


def gemm_timelines(which: str, tokens: list[int]) -> None:
    """Where a decode-size GEMM call's time goes: %globaltimer stamps that every block of the
    kernel writes (ops.linear.gemm_timeline), read after a CUDA-graph loop of calls on rotating
    weights. One JSON line per (shape, tokens): microseconds after the first block's entry, as
    [fastest, median, slowest] over the blocks."""
    import torch

    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05, gemm_timeline

    c = QWEN3_8B
    shapes = {
        "qkv": ((c["num_attention_heads"] + 2 * c["num_key_value_heads"]) * c["head_dim"], c["hidden_size"]),
        "o": (c["hidden_size"], c["num_attention_heads"] * c["head_dim"]),
        "gate_up": (2 * c["intermediate_size"], c["hidden_size"]), "down": (c["hidden_size"], c["intermediate_size"]),
    }  # fmt: skip
    names = ["entry", "setup", "wait_over", "first_stage", "last_mma", "last_accumulator", "epilogue_done"]
    for name, (N, K) in shapes.items():
        if which not in ("all", name):
            continue
        ws = [(torch.randn(N, K, device="cuda") * 0.02).bfloat16() for _ in range(6)]
        for M in tokens:
            x = torch.randn(M, K, device="cuda").bfloat16()
            stamps = torch.zeros(160, 8, dtype=torch.int64, device="cuda")
            for i in range(3):
                gemm_tcgen05(x, ws[i], None, torch.bfloat16)
            torch.cuda.synchronize()
            gemm_timeline(stamps)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for i in range(12):
                    gemm_tcgen05(x, ws[i % 6], None, torch.bfloat16)
            gemm_timeline(None)
            stamps.zero_()
            graph.replay()
            torch.cuda.synchronize()
            check_gemm_status()
            host = stamps.cpu()
            blocks = int(((host[:, 0] > 0) & (host[:, 3] > 0)).sum())  # a block's row has a first-stage stamp
            per_block, reduction = host[:blocks].double(), host[blocks].double()  # then the reduction's three stamps
            t0 = per_block[:, 0].min()
            line = {"gemm": name, "tokens": M, "blocks": blocks}
            for i, n in enumerate(names):
                col = (per_block[:, i] - t0) / 1000.0
                line[n] = [round(float(col.min()), 2), round(float(col.median()), 2), round(float(col.max()), 2)]
            if reduction[1] > 0:
                line["reduction"] = {k: round(float((reduction[i] - t0) / 1000.0), 2) for i, k in enumerate(["entry", "wait_over", "end"])}
            print(json.dumps(line))
        del ws


def reference_arm(args) -> int:
    """The same measurement on the unmodified reference (baseline/reference_arm.py): its own
    engine, sampler and PyTorch model code on this GPU, nothing of this package."""
    from baseline.reference_arm import ReferenceUnavailable, run

    shape = SHAPES[args.shape]
    layers = args.layers if args.layers_given else shape["num_hidden_layers"]
    warmup = max(args.warmup, 3)
    try:
        with ClockSampler("reference_clocks.csv") as clocks:
            r = run(shape, layers, args.batch, args.steps, warmup, PROMPT_TOKENS, CONTEXT, BLOCK_SIZE)
    except ReferenceUnavailable as why:
        print(json.dumps({"impl": "reference", "unavailable": str(why)}))
        return 0
    pk = peaks()
    c = shape
    flops = prefill_flops(argparse.Namespace(
        num_attention_heads=c["num_attention_heads"], num_key_value_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
        hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"], num_hidden_layers=layers, vocab_size=c["vocab_size"],
    ), PROMPT_TOKENS)  # fmt: skip
    main_, ms = r["main"], r["main"]["device_ms"]
    line = {
        "impl": "reference",
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, context 2048-4096); prefill tok/s at 2,048 tokens",
        "value": round(main_["tokens_per_s_device"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {
            "model": "Qwen3-8B shape", "layers": layers, "layers_full": shape["num_hidden_layers"], "hidden": c["hidden_size"],
            "heads": c["num_attention_heads"], "kv_heads": c["num_key_value_heads"], "head_dim": c["head_dim"],
            "intermediate": c["intermediate_size"], "vocab": c["vocab_size"], "global_batch": args.batch, "seq_len": CONTEXT,
            "prompt_tokens": PROMPT_TOKENS, "block_size": BLOCK_SIZE, "parallelism": "single-gpu",
            "l2": "weights read per step exceed L2; no flush needed", "sampling": "greedy",
            "path": "the reference's Engine.step on cuda: PyTorch matmul, SDPA, its own sampler",
        },
        "e2e": {"value": round(main_["tokens_per_s_e2e"], 1), "unit": "tokens/s"},
        "prefill": {"value": round(PROMPT_TOKENS * 1000.0 / r["prefill_ms"], 1), "tokens": PROMPT_TOKENS, "ms": round(r["prefill_ms"], 3),
                    "frac": round(flops / (r["prefill_ms"] * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "budget512_ms": round(r["prefill_budget512_ms"], 3)},
        "points": r["points"],
        "clocks": clocks.summary(),
    }  # fmt: skip
    print(json.dumps(line))
    return 0


def main() -> int:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=64)
    parser.add_argument("--warmup", type=int, default=8)
    parser.add_argument("--layers", type=int, default=QWEN3_8B["num_hidden_layers"],
                        help="fewer layers than the model has (same layer sizes), where time or memory needs it")  # fmt: skip
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--only", choices=["decode", "prefill", "gemm", "serve", "attention", "sampling"], help="time just this (for profiling small cases and the other shapes)")
    parser.add_argument("--shape", default="8b", choices=sorted(SHAPES), help="with --only decode/prefill/serve: layer sizes of Qwen3-8B, -14B or -32B")
    parser.add_argument("--context", type=int, default=PROMPT_TOKENS, help="with --only decode: tokens each request holds when decoding starts")
    parser.add_argument("--requests", type=int, default=32, help="with --only serve: requests submitted at once")
    parser.add_argument("--decode-tokens", type=int, default=256, help="with --only serve: tokens generated per request")
    parser.add_argument("--budget", type=int, default=512, help="with --only serve: the scheduler's token budget per step")
    parser.add_argument("--gemm-shape", default="all", help="with --only gemm: qkv, o, gate_up, down, lm_head or all")
    parser.add_argument("--gemm-tokens", default="1,8,64,2048", help="with --only gemm: token counts, comma-separated")
    parser.add_argument("--timeline", action="store_true", help="with --only gemm: where a decode-size call's time goes")
    args = parser.parse_args()
    args.layers_given = any(a == "--layers" or a.startswith("--layers=") for a in sys.argv[1:])
    if args.gpus != 1:
        print(f"bench.py measures one GPU; --gpus {args.gpus} is not supported (the engine is single-GPU)")
        return 2
    if args.impl == "reference":
        return reference_arm(args)
    warmup = max(args.warmup, 3)

    import torch

    from atomserve_b200.ops import require_device

    require_device()
    pk = peaks()
    if args.only == "attention":
        attention_partition_sweep([4, 8, 16, 32, 64, 128], [2048, 8192])
        return 0
    if args.only == "sampling":
        time_sampling([1, 8, 64], SHAPES[args.shape]["vocab_size"])
        return 0
    if args.only == "gemm" and args.timeline:
        gemm_timelines(args.gemm_shape, [int(t) for t in args.gemm_tokens.split(",")])
        return 0
    if args.only == "gemm":
        time_gemms(args.gemm_shape, [int(t) for t in args.gemm_tokens.split(",")], max(args.steps // 4, 4))
        return 0
    shape = SHAPES[args.shape]
    layers = args.layers if args.layers_given else shape["num_hidden_layers"]
    if args.only == "serve":
        config, model, engine = build_engine(layers, max_seqs=args.requests, shape=shape,
                                             context=2048 + args.decode_tokens + BLOCK_SIZE, budget=args.budget)  # fmt: skip
        result = time_serving(engine, args.requests, args.decode_tokens)
        print(json.dumps({"only": "serve", "shape": args.shape, "layers": layers, "layers_full": shape["num_hidden_layers"],
                          "budget": args.budget, **result}))  # fmt: skip
        return 0
    if args.only == "decode":
        context = args.context + warmup + args.steps + args.batch + 64
        config, model, engine = build_engine(layers, max_seqs=max(args.batch, 8), shape=shape,
                                             context=-(-context // BLOCK_SIZE) * BLOCK_SIZE, budget=max(args.context, PROMPT_TOKENS))  # fmt: skip
        ms, launches, ctx, e2e, _ = time_decode(engine, args.batch, args.steps, warmup, args.context)
        gbs = step_bytes(config, args.batch, ctx) / (ms * 1e-3) / 1e9
        print(json.dumps({"only": "decode", "shape": args.shape, "batch": args.batch, "layers": layers,
                          "layers_full": shape["num_hidden_layers"], "context": ctx, "ms_per_step": round(ms, 4),
                          "tokens_per_s": round(args.batch * 1000.0 / ms, 1), "e2e_tokens_per_s": round(e2e, 1),
                          "gbs": round(gbs, 1), "hbm_frac": round(gbs / pk["hbm_gbs"], 4), "gpu_launches": launches}))  # fmt: skip
        return 0
    config, model, engine = build_engine(layers, max_seqs=64, shape=shape)
    if args.only == "prefill":
        ms = time_prefill(engine, steps=args.steps, warmup=warmup)
        print(json.dumps({"only": "prefill", "layers": layers, "tokens": PROMPT_TOKENS, "ms": round(ms, 3)}))
        return 0
    with ClockSampler() as clocks:
        device_ms, launches, ctx, e2e, upload_bytes = time_decode(engine, args.batch, args.steps, warmup)
    points = {}
    for b in (1, 64):
        ms, _, _, e, _ = time_decode(engine, b, max(args.steps // 2, 8), 3)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
        points[f"decode_b{b}_e2e"] = round(e, 1)
    # long enough for the power cap to act and for a few clock samples: the prefill runs at the cap
    with ClockSampler("bench_clocks_prefill.csv") as prefill_clocks:
        prefill_ms = time_prefill(engine, steps=20, warmup=3)
    prefill_512_ms = time_prefill_through_engine(model, 512, repeats=10, warmup=3)
    sampled_e2e, _ = time_e2e(engine, args.batch, max(args.steps // 2, 8), 3, PROMPT_TOKENS, greedy=False)
    points[f"decode_b{args.batch}_sampled_e2e"] = round(sampled_e2e, 1)

    value = args.batch * 1000.0 / device_ms
    achieved = step_bytes(config, args.batch, ctx) / (device_ms * 1e-3) / 1e9
    flops = prefill_flops(config, PROMPT_TOKENS)
    line = {
        "metric": "decode tok/s at batch 8 (Qwen3-8B shape, context 2048-4096); prefill tok/s at 2,048 tokens",
        "value": round(value, 1),
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": args.steps,
        "warmup": warmup,
        "ms_per_step": round(device_ms, 4),
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic token ids, random-init weights N(0, 0.02)",
        "config": {
            "model": "Qwen3-8B shape", "layers": layers, "layers_full": QWEN3_8B["num_hidden_layers"],
            "hidden": config.hidden_size, "heads": config.num_attention_heads, "kv_heads": config.num_key_value_heads,
            "head_dim": config.head_dim, "intermediate": config.intermediate_size, "vocab": config.vocab_size,
            "global_batch": args.batch, "seq_len": CONTEXT, "prompt_tokens": PROMPT_TOKENS, "block_size": BLOCK_SIZE,
            "parallelism": "single-gpu", "l2": "weights read per step exceed L2; no flush needed", "sampling": "greedy",
        },
        "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": upload_bytes,
                "d2h_bytes_per_step": 4 * args.batch},
        "gpu_launches": launches * 1,
        "prefill": {"value": round(PROMPT_TOKENS * 1000.0 / prefill_ms, 1), "tokens": PROMPT_TOKENS, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "frac_sustained": round(flops / (prefill_ms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4),
                    "sm_mhz": prefill_clocks.summary()["sm_mhz"], "budget512_ms": round(prefill_512_ms, 3)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "peaks": pk["source"]},
        "points": points,
        "clocks": clocks.summary(),
    }  # fmt: skip
    if layers == QWEN3_8B["num_hidden_layers"] and args.batch == 1:
        line["vs_baseline"] = round(value / PUBLISHED_8B_BATCH1, 2)
    elif "decode_b1" in points and layers == QWEN3_8B["num_hidden_layers"]:
        line["vs_baseline"] = round(points["decode_b1"] / PUBLISHED_8B_BATCH1, 2)
        line["vs_baseline_note"] = "decode_b1 over the reference's published Qwen3-8B batch-1 15.7 tok/s (M4 Pro)"
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
