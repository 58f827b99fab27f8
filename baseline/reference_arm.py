"""The reference arm of bench.py: aneesh-sathe/atomserve itself, unmodified, timed on this GPU.

The reference is written for Apple MPS, but its engine is plain PyTorch and follows the device
its weights are on: `create_engine` builds the pool on `weights.embed.device`
(atomserve/engine.py:254-259), `ModelRunner` turns its Metal kernels off by itself anywhere
else (atomserve/runner.py:82-84, atomserve/kernels.py:581-588). So this arm builds the
reference's own `Weights` from seeded random bfloat16 tensors on `cuda`, calls its own
`create_engine`, and times it by its own method (bench/engine.py:90-126): prompts of synthetic
ids, prefill steps untimed, decode steps timed, tokens counted, one cold prompt for the prefill.

A plain copy of the reference's `atomserve/` folder is expected under `baseline/_ref/` (its
`pip install` is not needed and fails here: the `uv_build` backend and Python >= 3.14 are not
in this image). Its files are compiled with deferred annotations by an import hook, which is
all Python 3.12 needs to run them; nothing in them is changed. Nothing of atomserve_b200 is
imported here.
"""

from __future__ import annotations

import __future__ as _future

import dataclasses
import importlib.abc
import importlib.util
import pathlib
import sys
import time
import traceback

HERE = pathlib.Path(__file__).resolve().parent


class ReferenceUnavailable(RuntimeError):
    pass


def install_reference(root: pathlib.Path | None = None) -> pathlib.Path:
    """Make `import atomserve` find the unmodified copy under baseline/_ref."""
    root = root or HERE / "_ref"
    if not (root / "atomserve" / "engine.py").exists():
        raise ReferenceUnavailable(f"no copy of the reference's atomserve/ folder under {root.name}/ beside {pathlib.Path(__file__).name}")

    class Loader(importlib.abc.SourceLoader):
        def __init__(self, path):
            self.path = path

        def get_filename(self, name):
            return self.path

        def get_data(self, path):
            return pathlib.Path(path).read_bytes()

        def source_to_code(self, data, path, *, _optimize=-1):
            return compile(data, path, "exec", flags=_future.annotations.compiler_flag, dont_inherit=True)

    class Finder(importlib.abc.MetaPathFinder):
        def find_spec(self, name, path, target=None):
            if name != "atomserve" and not name.startswith("atomserve."):
                return None
            p = root.joinpath(*name.split("."))
            if p.is_dir():
                init = str(p / "__init__.py")
                return importlib.util.spec_from_file_location(name, init, loader=Loader(init), submodule_search_locations=[str(p)])
            f = p.with_suffix(".py")
            return importlib.util.spec_from_file_location(name, f, loader=Loader(str(f))) if f.exists() else None

    sys.meta_path.insert(0, Finder())
    return root


def random_weights(config: dict, seed: int, device: str):
    """The reference's own Weights / LayerWeights, N(0, 0.02) matrices and 1 + N(0, 0.1) gains
    in bfloat16 on the device, q|k|v and gate|up stacked as its loader stacks them
    (atomserve/loader.py:101-121)."""
    import torch
    from atomserve.model import LayerWeights, Weights

    g = torch.Generator(device=device).manual_seed(seed)
    d, hd = config["hidden_size"], config["head_dim"]
    H, KV, I, V = config["num_attention_heads"], config["num_key_value_heads"], config["intermediate_size"], config["vocab_size"]

    def matrix(rows, cols):
        return (torch.randn(rows, cols, device=device, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)

    def gain(n):
        return (1 + 0.1 * torch.randn(n, device=device, generator=g, dtype=torch.float32)).to(torch.bfloat16)

    layers = [
        LayerWeights(
            input_norm=gain(d), qkv_proj=matrix((H + 2 * KV) * hd, d), q_norm=gain(hd), k_norm=gain(hd),
            o_proj=matrix(d, H * hd), post_attn_norm=gain(d), gate_up_proj=matrix(2 * I, d), down_proj=matrix(d, I),
        )
        for _ in range(config["num_hidden_layers"])
    ]  # fmt: skip
    embed = matrix(V, d)
    head = embed if config.get("tie_word_embeddings") else matrix(V, d)
    return Weights(embed=embed, layers=layers, final_norm=gain(d), lm_head=head)


def prompts(batch: int, length: int) -> list[list[int]]:
    """bench/engine.py:90-92."""
    return [[(1000 + 37 * b + i) % 150000 for i in range(length)] for b in range(batch)]


def time_decode(engine, batch: int, prompt_tokens: int, steps: int, warmup: int, greedy: bool = True, passes: int = 2) -> dict:
    """The faster of `passes` identical runs of `decode_pass`. The first run at a batch size pays,
    in every step, for whatever the libraries under PyTorch set up once per new shape (the
    attention call sees a context one token longer each step: 53 ms a step on the first run
    against 13 ms on the second, batch 8, measured on a B200); a server meets each shape again
    and again, so the warmed run is the reference's speed."""
    runs = [decode_pass(engine, batch, prompt_tokens, steps, warmup, greedy) for _ in range(passes)]
    return min(runs, key=lambda r: r["device_ms"])


def decode_pass(engine, batch: int, prompt_tokens: int, steps: int, warmup: int, greedy: bool = True) -> dict:
    """bench/engine.py:95-118 with CUDA events beside the wall clock: prefill until every request
    has its first token (untimed), `warmup` decode steps, then `steps` timed Engine.step() calls
    (host token ids in, sampled ids out, each step)."""
    import torch
    from atomserve.sequence import THINKING_PARAMS, SamplingParams

    base = SamplingParams(temperature=0.0) if greedy else THINKING_PARAMS
    params = dataclasses.replace(base, max_tokens=warmup + steps + 8, ignore_eos=True)
    handles = [engine.submit(p, params) for p in prompts(batch, prompt_tokens)]
    while any(h.first_token_at is None for h in handles):
        engine.step()
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    before = engine.num_generated_tokens
    t0 = time.perf_counter()
    start.record()
    for _ in range(steps):
        engine.step()
    end.record()
    torch.cuda.synchronize()
    seconds = time.perf_counter() - t0
    tokens = engine.num_generated_tokens - before
    device_ms = start.elapsed_time(end) / steps
    while engine.step():
        pass
    for h in handles:
        list(h)
    return {"device_ms": device_ms, "tokens_per_s_device": tokens / (device_ms * steps * 1e-3), "tokens_per_s_e2e": tokens / seconds}


def time_prefill(engine, prompt_tokens: int, repeats: int, warmup: int) -> float:
    """bench/engine.py:121-126: one cold prompt, one output token; milliseconds, CUDA events."""
    import torch
    from atomserve.sequence import SamplingParams

    params = SamplingParams(temperature=0.0, max_tokens=1)
    for _ in range(warmup):
        engine.generate(prompts(1, prompt_tokens), params)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(repeats):
        engine.generate(prompts(1, prompt_tokens), params)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / repeats


def run(shape: dict, layers: int, batch: int, steps: int, warmup: int, prompt_tokens: int, context: int, block_size: int) -> dict:
    """Everything the reference arm measures, as the fields of bench.py's line; raises
    ReferenceUnavailable with the failing line and message if the reference cannot run here."""
    try:
        install_reference()
        import torch

        if not torch.cuda.is_available():
            raise ReferenceUnavailable("no CUDA device")
        from atomserve.config import EngineConfig, ModelConfig
        from atomserve.engine import create_engine

        cfg = {**shape, "num_hidden_layers": layers}
        model_config = ModelConfig.from_dict(cfg)
        weights = random_weights(cfg, seed=0, device="cuda")

        def engine_for(max_seqs: int, budget: int):
            blocks = max_seqs * (context // block_size) + 64
            engine_config = EngineConfig(block_size=block_size, num_blocks=blocks, max_num_seqs=max_seqs,
                                         max_num_batched_tokens=budget, max_model_len=context,
                                         enable_prefix_caching=False)  # fmt: skip
            return create_engine(weights, model_config, engine_config, frozenset())

        engine = engine_for(max(64, batch), prompt_tokens)
        main = time_decode(engine, batch, prompt_tokens, steps, warmup)
        sampled = time_decode(engine, batch, prompt_tokens, max(steps // 2, 8), 3, greedy=False)
        points = {}
        for b in (1, 64):
            r = time_decode(engine, b, prompt_tokens, max(steps // 2, 8), 3)
            points[f"decode_b{b}"] = round(r["tokens_per_s_device"], 1)
            points[f"decode_b{b}_e2e"] = round(r["tokens_per_s_e2e"], 1)
        points[f"decode_b{batch}_sampled_e2e"] = round(sampled["tokens_per_s_e2e"], 1)
        prefill_ms = time_prefill(engine, prompt_tokens, repeats=5, warmup=2)
        del engine
        torch.cuda.empty_cache()
        chunked = engine_for(8, 512)  # the reference's default budget (atomserve/config.py:75): four portions
        prefill_512_ms = time_prefill(chunked, prompt_tokens, repeats=5, warmup=2)
        return {"main": main, "points": points, "prefill_ms": prefill_ms, "prefill_budget512_ms": prefill_512_ms}
    except ReferenceUnavailable:
        raise
    except Exception as error:  # noqa: BLE001  report where the reference stopped
        tb = traceback.extract_tb(error.__traceback__)
        inside = [f for f in tb if "_ref" in f.filename] or list(tb)
        where = inside[-1]
        raise ReferenceUnavailable(
            f"{pathlib.Path(where.filename).name}:{where.lineno} `{(where.line or '').strip()}` raised {type(error).__name__}: {str(error).splitlines()[0] if str(error) else ''}"
        ) from error
