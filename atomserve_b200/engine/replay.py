"""Trace replay: feed given token ids through the model step by step and write the logits.

It samples nothing and owns no model code: it loads the model as the engine does, builds the
same cache manager and runner, and for every step of the trace calls the runner's step
function with the rows the trace gives. What the trace decides (which tokens of which request
run in which step, and when a request ends) is all that the scheduler would otherwise decide.

Input, one JSON object per line on standard input:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

For a step that wants logits, `<out>/<step>.f32` holds them as little-endian float32
[wanted, vocab], in the order of the entries and of `want`. After every step the line
`done <step>` is printed and flushed.
"""

from __future__ import annotations

import argparse
import json
import sys
from pathlib import Path

import torch

from atomserve_b200.cache.manager import CacheManager, RequestCache
from atomserve_b200.engine.runner import ModelRunner, Row
from atomserve_b200.ops import require_device
from atomserve_b200.weights.loader import load_model, parse_dtype

MAX_LIVE_REQUESTS = 8


class TraceReplayer:
    def __init__(self, model_dir: str | Path, dtype: str, max_tokens: int, block_size: int = 16,
                 device: str = "cuda", cuda_graphs: bool = True, max_live: int = MAX_LIVE_REQUESTS):  # fmt: skip
        _, self.config, self.model = load_model(model_dir, dtype, device)
        requirements = self.model.cache_requirements()
        # --max-tokens counts what live requests hold, each rounded up to whole pages of 64
        # tokens; with pages of `block_size` (a divisor of 64) that is this many pages.
        num_blocks = -(-max_tokens // block_size)
        self.max_live = max_live  # requests that may hold pages and a state slot at once
        self.cache = CacheManager(requirements, block_size, num_blocks, max_live,
                                  parse_dtype(dtype), device)  # fmt: skip
        self.runner = ModelRunner(self.model, self.cache, cuda_graphs=cuda_graphs)
        self.live: dict[str, tuple[RequestCache, int]] = {}  # id -> (cache, tokens computed)

    def step(self, entries: list[dict], end: list) -> torch.Tensor:
        rows = []
        for e in entries:
            rid = str(e["id"])
            if rid not in self.live:
                rc = self.cache.new_request()
                if not self.cache.admit(rc):
                    raise RuntimeError(f"more than {self.max_live} requests are live")
                self.live[rid] = (rc, 0)
            rc, computed = self.live[rid]
            tokens = [int(t) for t in e["tokens"]]
            if not self.cache.reserve(rc, computed, len(tokens)):
                raise RuntimeError(
                    f"the cache pool ({self.cache.num_blocks} pages of {self.cache.block_size}) "
                    f"cannot hold {len(tokens)} more tokens of request {rid}"
                )
            rows.append(Row(tokens, computed, rc, [int(w) for w in e.get("want", [])]))
            self.live[rid] = (rc, computed + len(tokens))
        logits = self.runner.step(rows)
        if self.runner.device_status is not None:
            problem = self.runner.device_status.problem()  # a read of the device: replay is no hot path
            if problem:
                raise RuntimeError(f"step failed on the device: {problem}")
        for rid in end:
            rc, _ = self.live.pop(str(rid))
            self.cache.free(rc)
        return logits


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    parser.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    parser.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    parser.add_argument("--out", required=True, help="folder for <step>.f32 files")
    parser.add_argument("--max-tokens", type=int, required=True,
                        help="most tokens live requests hold at any time (sizes the cache pool)")  # fmt: skip
    parser.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    args = parser.parse_args(argv)
    require_device()
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    print("trace_run: loading model and kernels", file=sys.stderr, flush=True)
    from atomserve_b200.ops import library

    library.lib()  # compiles the kernels now if this checkout has no current build
    replayer = TraceReplayer(args.model, args.dtype, args.max_tokens, args.block_size)
    print("trace_run: ready", file=sys.stderr, flush=True)
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        record = json.loads(line)
        logits = replayer.step(record.get("entries", []), record.get("end", []))
        if logits.shape[0] > 0:
            data = logits.detach().to("cpu", torch.float32).contiguous().numpy().astype("<f4", copy=False)
            data.tofile(str(out / f"{record['step']}.f32"))
        print(f"done {record['step']}", flush=True)
    return 0
