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


class Oracle:
    """Logits of a whole prompt from the plain implementation, computed in float64 and kept as
    float32; indexing gives the rows asked for, still carrying the prompt's bfloat16 allowance.
    (Float64, because the plain implementation's own float32 rounding is of the size of the
    float32 tolerance: on a 230-token prompt of config E it lay 2.3e-5 of the largest logit from
    the float64 result at one position, where the engine's float32 path lay 0.8e-5 from it.)"""

    def __init__(self, w=None, cfg=None, prompt=None, logits=None, allowance=None):
        if logits is None:
            logits = plain.forward(w, cfg, prompt, dtype=torch.float64).float()
            allowance = bfloat16_tolerance(w, cfg, prompt, logits)
        self.logits, self.allowance = logits, allowance

    def __getitem__(self, rows):
        return Oracle(logits=self.logits[rows], allowance=self.allowance)


BF16_REPORT: list[tuple[str, float]] = []  # (what, error / allowance) of every bfloat16 check


def check(got, oracle, dtype, what):
    ref = oracle.logits
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} for {tuple(ref.shape)}"
    if dtype == "float32":
        err = rel_error(got.cpu(), ref)
        assert err < FLOAT32_TOLERANCE, f"{what}: relative error {err:.3g}"
        assert torch.equal(got.cpu().argmax(-1), ref.argmax(-1)), what
    else:
        err = float((got.cpu() - ref).abs().max())
        assert err <= oracle.allowance, f"{what}: error {err:.3g}, allowed {oracle.allowance:.3g}"
        BF16_REPORT.append((what, err / oracle.allowance))


def mixed_trace(ps, rng, max_live=4, largest=20):
    """Steps that keep up to `max_live` requests going: each live request brings a portion of
    random size, 2 to `largest` - 1 tokens (prompt phase) or one token (its last 8 tokens), some sit a step out."""
    steps, live, waiting, done_at = [], {}, list(range(len(ps))), {}
    while waiting or live:
        while waiting and len(live) < max_live:
            live[waiting.pop(0)] = 0
        entries, end = [], []
        for i in list(live):
            if len(live) > 1 and rng.random() < 0.2:
                continue
            at, total = live[i], len(ps[i])
            n = 1 if at >= total - 8 else min(int(rng.integers(2, largest)), total - 8 - at) or 1
            entries.append(dict(id=i, tokens=ps[i][at : at + n], want=list(range(n)), at=at))
            live[i] = at + n
            if at + n == total:
                end.append(i)
                del live[i]
        if entries:
            steps.append((entries, end))
    return steps


def assert_near_best_tokens(w: dict, cfg: dict, prompt: list[int], out: list[int], what: str = "") -> None:
    """Judge greedy tokens of a bfloat16 engine: bfloat16 may break near-ties differently, so
    each chosen token is held against the oracle run on the engine's own sequence: its logit must
    lie within twice the bfloat16 allowance of the best one at that position."""
    full = list(prompt) + list(out)
    ref = plain.forward(w, cfg, full)
    allowance = bfloat16_tolerance(w, cfg, full, ref)
    for i, token in enumerate(out):
        row = ref[len(prompt) + i - 1]
        gap = float(row.max() - row[token])
        assert gap <= 2 * allowance, f"{what} token {i} ({token}) lies {gap:.3g} below the best, allowed {2 * allowance:.3g}"
