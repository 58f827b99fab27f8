"""The sampler: next-token logits to chosen tokens, for a whole batch at once.

    logits -> presence penalty -> top-k -> / temperature -> softmax -> top-p -> draw

Every row has its own settings, handed to the kernel as per-row arrays in one upload
(atomserve/sampler.py:82-141 is the reference's pipeline; the kernel in csrc/sampling.cu
applies the same rules without sorting). A batch of greedy rows is a single argmax kernel.

Random streams: each request draws from Philox keyed by its own seed (the request's `seed`,
or one derived from the sampler's base seed and the request id) with the number of tokens it
has generated as the counter. What a request draws therefore never depends on its batch
neighbours, and a preempted request that is recomputed draws the same tokens again.
"""

from __future__ import annotations

import os

import torch

from atomserve_b200 import ops
from atomserve_b200.engine.sequence import Sequence

_MASK63 = (1 << 63) - 1


class Sampler:
    def __init__(self, device: torch.device | str, base_seed: int | None = None):
        self.device = torch.device(device)
        self.base_seed = base_seed if base_seed is not None else int.from_bytes(os.urandom(8), "little")
        self._host: torch.Tensor | None = None  # the per-row settings of a step, packed for one upload
        self._dev: torch.Tensor | None = None

    def seed_of(self, seq: Sequence) -> int:
        if seq.params.seed is not None:
            return seq.params.seed & _MASK63
        return (self.base_seed * 0x9E3779B97F4A7C15 + seq.id * 0xBF58476D1CE4E5B9 + 1) & _MASK63

    def release(self, seq_id: int) -> None:
        """Nothing is kept per request: seeds and counters derive from the request itself."""

    def sample(self, logits: torch.Tensor, seqs: list[Sequence]) -> list[int]:
        """One token per row; logits [B, vocab] float32, row i belongs to seqs[i]. The read
        of the result is the step's one device synchronisation."""
        if not seqs:
            return []
        self._apply_presence_penalty(logits, seqs)
        if all(s.params.temperature == 0 for s in seqs):
            return ops.argmax_rows(logits).tolist()
        n = len(seqs)
        # One upload from pinned memory: four rows of n 64-bit words, seeds, draw counters, then
        # temperatures and top-p as the float32 halves of the third row, top-k as int32 in the fourth.
        # (The previous step's upload has left the host buffer: that step ended with a read of its result.)
        if self._host is None or self._host.shape[0] < 4 * n:
            cap = max(4 * n, 1024)
            self._host = torch.empty(cap, dtype=torch.int64, pin_memory=self.device.type == "cuda")
            self._dev = torch.empty(cap, dtype=torch.int64, device=self.device)
        host, dev = self._host[: 4 * n].view(4, n), self._dev[: 4 * n].view(4, n)
        host[0] = torch.tensor([self.seed_of(s) for s in seqs], dtype=torch.int64)
        host[1] = torch.tensor([len(s.token_ids) - s.num_prompt_tokens for s in seqs], dtype=torch.int64)
        floats = host[2].view(torch.float32)
        floats[:n] = torch.tensor([s.params.temperature for s in seqs], dtype=torch.float32)
        floats[n:] = torch.tensor([s.params.top_p for s in seqs], dtype=torch.float32)
        host[3].view(torch.int32)[:n] = torch.tensor([s.params.top_k for s in seqs], dtype=torch.int32)
        dev.copy_(host, non_blocking=True)
        dev_floats = dev[2].view(torch.float32)
        out = ops.sample_rows(logits, dev_floats[:n], dev[3].view(torch.int32)[:n], dev_floats[n:], dev[0], dev[1])
        assert out.shape[0] == n
        return out.tolist()

    def _apply_presence_penalty(self, logits: torch.Tensor, seqs: list[Sequence]) -> None:
        rows, tokens, amounts = [], [], []
        for i, seq in enumerate(seqs):
            if seq.params.presence_penalty != 0:
                seen = set(seq.output_ids)
                rows.extend([i] * len(seen))
                tokens.extend(seen)
                amounts.extend([seq.params.presence_penalty] * len(seen))
        if rows:
            ints = torch.tensor([rows, tokens], dtype=torch.int32).to(self.device)
            ops.presence_penalty(logits, ints[0], ints[1], torch.tensor(amounts, dtype=torch.float32).to(self.device))
