"""Sampling kernels over float32 logits [B, V]."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, lib, ptr, require_cuda, stream


def _logits(logits: torch.Tensor) -> None:
    require_cuda(logits)
    if logits.dim() != 2 or logits.dtype != torch.float32 or not logits.is_contiguous():
        raise KernelLibraryError("sampling takes contiguous float32 logits [rows, vocab]")


def argmax_rows(logits: torch.Tensor) -> torch.Tensor:
    """The largest logit's token id per row, the lowest id among equals: int32 [B]."""
    _logits(logits)
    out = torch.empty(logits.shape[0], device=logits.device, dtype=torch.int32)
    check(lib().asb_argmax_rows(ptr(out), ptr(logits), logits.shape[0], logits.shape[1], stream()))
    return out


def presence_penalty(logits: torch.Tensor, rows: torch.Tensor, tokens: torch.Tensor, amounts: torch.Tensor) -> None:
    """In place: logits[rows[i], tokens[i]] -= amounts[i]; each (row, token) pair appears once."""
    _logits(logits)
    require_cuda(rows, tokens, amounts)
    if rows.dtype != torch.int32 or tokens.dtype != torch.int32 or amounts.dtype != torch.float32:
        raise KernelLibraryError("presence_penalty takes int32 rows and tokens and float32 amounts")
    check(lib().asb_presence_penalty(ptr(logits), ptr(rows), ptr(tokens), ptr(amounts), rows.shape[0],
                                     logits.shape[1], stream()))  # fmt: skip


def sample_rows(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
                seed: torch.Tensor, counter: torch.Tensor) -> torch.Tensor:  # fmt: skip
    """One token per row. temperature, top_p: float32 [B]; top_k: int32 [B] (0: all); seed,
    counter: int64 [B]. A row with temperature 0 gets its argmax."""
    _logits(logits)
    require_cuda(temperature, top_k, top_p, seed, counter)
    B = logits.shape[0]
    for t, dt in ((temperature, torch.float32), (top_k, torch.int32), (top_p, torch.float32),
                  (seed, torch.int64), (counter, torch.int64)):  # fmt: skip
        if t.dtype != dt or t.shape != (B,) or not t.is_contiguous():
            raise KernelLibraryError(f"sample_rows: a per-row setting has dtype {t.dtype}, shape {tuple(t.shape)}")
    out = torch.empty(B, device=logits.device, dtype=torch.int32)
    check(lib().asb_sample_rows(ptr(out), ptr(logits), B, logits.shape[1], ptr(temperature), ptr(top_k),
                                ptr(top_p), ptr(seed), ptr(counter), stream()))  # fmt: skip
    return out
