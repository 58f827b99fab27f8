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
        floats = torch.tensor(
            [[s.params.temperature for s in seqs], [s.params.top_p for s in seqs]], dtype=torch.float32
        )
        top_k = torch.tensor([s.params.top_k for s in seqs], dtype=torch.int32)
        keys = torch.tensor([[self.seed_of(s) for s in seqs], [s.num_tokens - s.num_prompt_tokens for s in seqs]], dtype=torch.int64)
        floats, top_k, keys = (t.to(self.device, non_blocking=True) for t in (floats, top_k, keys))
        out = ops.sample_rows(logits, floats[0], top_k, floats[1], keys[0], keys[1])
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
