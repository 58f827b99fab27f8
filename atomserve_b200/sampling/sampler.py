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


class Picked:
    """A step's sampled ids on their way to the host: on the device (where the next step can take
    them as its input without waiting), and in pinned host memory once `arrived` has passed."""

    __slots__ = ("device_ids", "host_ids", "arrived")

    def __init__(self, device_ids: torch.Tensor, host_ids: torch.Tensor, arrived):
        self.device_ids, self.host_ids, self.arrived = device_ids, host_ids, arrived


class Sampler:
    def __init__(self, device: torch.device | str, base_seed: int | None = None):
        self.device = torch.device(device)
        self.base_seed = base_seed if base_seed is not None else int.from_bytes(os.urandom(8), "little")
        # Two sets of host buffers, used in turn: a step may be launched while the step before it
        # has not been read yet, and that step's uploads and results still own their buffers.
        self._turn = 0
        self._host: list[torch.Tensor | None] = [None, None]  # per-row settings, packed for one upload
        self._ids: list[torch.Tensor | None] = [None, None]   # the sampled ids, pinned
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
        return self.collect(self.launch(logits, seqs))

    def launch(self, logits: torch.Tensor, seqs: list[Sequence], ahead: int = 0) -> Picked:
        """Start the sampling of one token per row and the copy of the ids to the host; nothing
        waits. `ahead`: tokens each request will have gained, beyond those its list shows, by the
        time this step's token is drawn (1 for a step launched before its predecessor was read):
        it only moves the draw counters. Presence penalties need the list itself, so a step with
        one is not launched ahead."""
        if ahead and any(s.params.presence_penalty != 0 for s in seqs):
            raise ValueError("a step with presence penalties cannot be sampled ahead of its predecessor's tokens")
        self._turn ^= 1
        turn, n = self._turn, len(seqs)
        self._apply_presence_penalty(logits, seqs)
        if all(s.params.temperature == 0 for s in seqs):
            out = ops.argmax_rows(logits)
        else:
            # One upload from pinned memory: four rows of n 64-bit words, seeds, draw counters, then
            # temperatures and top-p as the float32 halves of the third row, top-k as int32 in the fourth.
            if self._host[turn] is None or self._host[turn].shape[0] < 4 * n:
                cap = max(4 * n, 1024)
                self._host[turn] = torch.empty(cap, dtype=torch.int64, pin_memory=self.device.type == "cuda")
            if self._dev is None or self._dev.shape[0] < 4 * n:
                self._dev = torch.empty(max(4 * n, 1024), dtype=torch.int64, device=self.device)
            host, dev = self._host[turn][: 4 * n].view(4, n), self._dev[: 4 * n].view(4, n)
            host[0] = torch.tensor([self.seed_of(s) for s in seqs], dtype=torch.int64)
            host[1] = torch.tensor([len(s.token_ids) - s.num_prompt_tokens + ahead for s in seqs], dtype=torch.int64)
            floats = host[2].view(torch.float32)
            floats[:n] = torch.tensor([s.params.temperature for s in seqs], dtype=torch.float32)
            floats[n:] = torch.tensor([s.params.top_p for s in seqs], dtype=torch.float32)
            host[3].view(torch.int32)[:n] = torch.tensor([s.params.top_k for s in seqs], dtype=torch.int32)
            dev.copy_(host, non_blocking=True)
            dev_floats = dev[2].view(torch.float32)
            out = ops.sample_rows(logits, dev_floats[:n], dev[3].view(torch.int32)[:n], dev_floats[n:], dev[0], dev[1])
        assert out.shape[0] == n
        if self.device.type != "cuda":
            return Picked(out, out, None)
        if self._ids[turn] is None or self._ids[turn].shape[0] < n:
            self._ids[turn] = torch.empty(max(n, 256), dtype=torch.int32, pin_memory=True)
        host_ids = self._ids[turn][:n]
        host_ids.copy_(out, non_blocking=True)
        arrived = torch.cuda.Event()
        arrived.record()
        return Picked(out, host_ids, arrived)

    def collect(self, picked: Picked) -> list[int]:
        """The ids of a launched step; waits for them (the step's one device synchronisation)."""
        if picked.arrived is not None:
            picked.arrived.synchronize()
        return picked.host_ids.tolist()

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
