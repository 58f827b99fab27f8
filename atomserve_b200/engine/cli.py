"""Command line: `python -m atomserve_b200 <model_dir>` loads a model folder and generates
token ids for the prompts given, through the engine.

It parses arguments and wires the pieces; it owns no inference logic
(atomserve/cli.py:34-200). Options the reference has keep their names and meanings: `model`,
`--dtype {bf16,fp32}`, `--kv-mem-gb`, `--block-size`, `--max-num-seqs`,
`--max-batched-tokens`, `--no-prefix-caching`, `--version`. The reference then serves HTTP and
a chat prompt; this engine deals in token ids, so prompts come as ids (`--prompt-ids`,
`--prompt-file`) with the request's sampling options, and results are printed as JSON lines.
"""

from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

import torch

from atomserve_b200 import __version__
from atomserve_b200.cache.manager import CacheManager
from atomserve_b200.config.engine_config import EngineConfig
from atomserve_b200.config.registry import load_model_config
from atomserve_b200.engine.engine import create_engine
from atomserve_b200.engine.sequence import SamplingParams
from atomserve_b200.ops import require_device
from atomserve_b200.parts.model import build_model
from atomserve_b200.weights.loader import load_tensors_into, read_eos_token_ids
from atomserve_b200.weights.random_init import RandomTensors, write_model_folder

DTYPES = {"bf16": torch.bfloat16, "fp32": torch.float32}


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(
        prog="atomserve_b200",
        description="Generate token ids from a model folder (config.json + safetensors) on one B200.",
        formatter_class=argparse.ArgumentDefaultsHelpFormatter,
    )
    parser.add_argument("model", help="local model directory (config.json, *.safetensors)")
    parser.add_argument("--dtype", choices=DTYPES, default="bf16", help="weights, activations and the KV cache")
    parser.add_argument("--kv-mem-gb", type=float, default=4.0, help="GiB of memory for the KV cache")
    parser.add_argument("--block-size", type=int, default=16, help="tokens per KV block")
    parser.add_argument("--max-num-seqs", type=int, default=32, help="most requests running at once")
    parser.add_argument("--max-batched-tokens", type=int, default=512,
                        help="token budget of one forward pass; smaller bounds the stall a long prompt "
                        "causes running streams, larger prefills a little faster")  # fmt: skip
    parser.add_argument("--no-prefix-caching", action="store_true", help="always recompute shared prompt prefixes")
    parser.add_argument("--version", action="version", version=f"%(prog)s {__version__}")
    # what takes the place of the reference's chat clients: prompts as token ids
    parser.add_argument("--prompt-ids", action="append", default=[], metavar="IDS",
                        help="a prompt as comma-separated token ids (repeatable)")  # fmt: skip
    parser.add_argument("--prompt-file", help="file with one JSON list of token ids per line")
    parser.add_argument("--max-tokens", type=int, default=64, help="tokens to generate per prompt")
    parser.add_argument("--temperature", type=float, default=0.6, help="0 is greedy")
    parser.add_argument("--top-k", type=int, default=20, help="0 disables")
    parser.add_argument("--top-p", type=float, default=0.95)
    parser.add_argument("--presence-penalty", type=float, default=0.0)
    parser.add_argument("--seed", type=int, default=None, help="seed of every request's random stream")
    parser.add_argument("--ignore-eos", action="store_true", help="generate past end-of-sequence tokens")
    parser.add_argument("--random-weights", type=int, default=None, metavar="SEED",
                        help="ignore the folder's safetensors and draw weights from this seed")  # fmt: skip
    parser.add_argument("--save-random-model", metavar="DIR",
                        help="with --random-weights: write config.json and model.safetensors to DIR and exit")  # fmt: skip
    parser.add_argument("--no-cuda-graphs", action="store_true", help="run decode steps eagerly")
    return parser


def engine_config_for(args: argparse.Namespace, model, max_positions: int) -> EngineConfig:
    """Size the cache pool from the memory budget; cap the sequence length by pool and model
    (atomserve/cli.py:99-119)."""
    block_bytes = CacheManager.bytes_per_block(model.cache_requirements(), args.block_size, DTYPES[args.dtype])
    num_blocks = int(args.kv_mem_gb * 2**30 // block_bytes)
    return EngineConfig(
        block_size=args.block_size,
        num_blocks=num_blocks,
        max_num_seqs=args.max_num_seqs,
        max_num_batched_tokens=args.max_batched_tokens,
        max_model_len=min(max_positions, num_blocks * args.block_size),
        enable_prefix_caching=not args.no_prefix_caching,
        cuda_graphs=not args.no_cuda_graphs,
    )


def read_prompts(args: argparse.Namespace) -> list[list[int]]:
    prompts = [[int(t) for t in text.split(",") if t.strip()] for text in args.prompt_ids]
    if args.prompt_file:
        for line in Path(args.prompt_file).read_text().splitlines():
            if line.strip():
                prompts.append([int(t) for t in json.loads(line)])
    return prompts


def main(argv: list[str] | None = None) -> int:
    args = build_parser().parse_args(argv)
    start = time.perf_counter()
    model_dir = Path(args.model).expanduser()
    if not model_dir.is_dir():
        print(f"atomserve_b200: {args.model} is not a local model directory", file=sys.stderr)
        return 1
    arch, config = load_model_config(model_dir)
    if args.save_random_model:
        if args.random_weights is None:
            print("atomserve_b200: --save-random-model needs --random-weights SEED", file=sys.stderr)
            return 1
        out = write_model_folder(config, args.random_weights, args.save_random_model,
                                 "bfloat16" if args.dtype == "bf16" else "float32")  # fmt: skip
        print(f"wrote {out}")
        return 0
    require_device()
    print(f"Loading {args.model} ({args.dtype}, cuda) ...", file=sys.stderr, flush=True)
    model = build_model(arch.build_spec(config))
    if args.random_weights is not None:
        model.load(RandomTensors(model.tensor_specs(), args.random_weights, DTYPES[args.dtype], "cuda"))
    else:
        load_tensors_into(model, model_dir, DTYPES[args.dtype], "cuda")
    engine_config = engine_config_for(args, model, model.spec.max_positions)
    engine = create_engine(model, engine_config, read_eos_token_ids(model_dir))
    # the first run builds kernels' lazy state and captures graphs: pay that before the prompts
    engine.generate([[0]], SamplingParams(temperature=0.0, max_tokens=2, ignore_eos=True))
    print(
        f"Ready in {time.perf_counter() - start:.1f}s. KV cache: "
        f"{engine_config.num_blocks * engine_config.block_size:,} tokens, "
        f"context up to {engine_config.max_model_len:,}.",
        file=sys.stderr, flush=True,
    )  # fmt: skip
    prompts = read_prompts(args)
    if not prompts:
        print("atomserve_b200: no prompts given (--prompt-ids or --prompt-file)", file=sys.stderr)
        return 0
    params = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p,
        presence_penalty=args.presence_penalty, max_tokens=args.max_tokens, seed=args.seed,
        ignore_eos=args.ignore_eos,
    )  # fmt: skip
    handles = [engine.submit(p, params) for p in prompts]
    while engine.step():
        pass
    for i, h in enumerate(handles):
        ids = list(h)
        print(json.dumps({"request": i, "output_ids": ids, "finish_reason": h.finish_reason}), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
