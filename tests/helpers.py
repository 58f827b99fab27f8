"""Test-side helpers: model folders from the plain generator, and ways of cutting requests
into replay steps. Nothing here is imported by the package."""

from __future__ import annotations

import json
import pathlib

import torch
from safetensors.torch import save_file

import plain_qwen3 as plain


def checkpoint(cfg: dict, seed: int, sharp: bool = True, bf16_exact: bool = True) -> dict:
    """Random float32 checkpoint. `sharp` multiplies the q/k norm gains by 2.5 so that
    attention scores spread over several units and single keys matter (with small random
    weights attention is nearly uniform and a misplaced key would hide in the average).
    `bf16_exact` rounds the matrices to bfloat16 values, so that a bfloat16 engine and the
    float32 oracle compute with the same weights."""
    w = plain.random_checkpoint(cfg, seed)
    for name in w:
        if sharp and (name.endswith("q_norm.weight") or name.endswith("k_norm.weight")):
            w[name] = w[name] * 2.5
        if bf16_exact and w[name].dim() == 2:
            w[name] = w[name].bfloat16().float()
    return w


def write_folder(cfg: dict, w: dict, folder: pathlib.Path) -> pathlib.Path:
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return folder


def prompts(cfg: dict, lengths: list[int], seed: int) -> list[list[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab_size"], (n,), generator=g).tolist() for n in lengths]


def rel_error(got: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest absolute difference over the largest reference magnitude."""
    return float((got.double() - ref.double()).abs().max() / ref.double().abs().max())


FLOAT32_TOLERANCE = 2e-5


def bfloat16_tolerance(w: dict, cfg: dict, prompt: list[int], ref: torch.Tensor) -> float:
    """How far (in absolute terms) bfloat16 logits may lie from the float32 oracle anywhere in
    this prompt. The yardstick is the plain implementation itself with every operation's result
    rounded to bfloat16: the engine rounds at fewer places and accumulates in float32, so its
    noise is of that size or smaller. Both are single draws of rounding noise, so the engine
    is allowed twice the yardstick's largest error, and never less than 1% of the prompt's
    largest logit. (What this cannot see, the float32 runs of the same tests do: they share
    every kernel and all host logic and are held to 2e-5.)"""
    rounded = plain.forward(w, cfg, prompt, activations=torch.bfloat16)
    return max(2 * float((rounded - ref).abs().max()), 0.01 * float(ref.abs().max()))
