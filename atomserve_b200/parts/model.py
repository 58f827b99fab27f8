"""A decoder assembled from a ModelSpec: embedding, the layers in their run order, final norm,
output head (atomserve/model.py:363-385 is the reference's fixed form of this loop)."""

from __future__ import annotations

import inspect

import torch

from atomserve_b200.parts.base import Block, CacheView, PageSpec, StateSpec, StepContext, build_block, build_part
from atomserve_b200.parts.spec import ModelSpec, TensorSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec):
        self.spec = spec
        d = spec.hidden_size
        self.embedding = build_part("embedding", spec.embedding, d)
        self.blocks: list[Block] = [
            build_block(
                layer.block,
                build_part("mixer", layer.mixer, d),
                build_part("feed_forward", layer.feed_forward, d),
                build_part("norm", layer.mixer_norm, d),
                build_part("norm", layer.feed_forward_norm, d),
            )
            for layer in spec.layers
        ]
        self.schedule = spec.schedule
        for i, call in enumerate(self.schedule):
            if not 0 <= call.layer < len(self.blocks):
                raise ValueError(f"run order entry {i} names layer {call.layer} of {len(self.blocks)}")
            if call.cache_from is not None:
                if not 0 <= call.cache_from < i or self.schedule[call.cache_from].cache_from is not None:
                    raise ValueError(f"run order entry {i} must read the cache of an earlier entry that owns one")
        self.final_norm = build_part("norm", spec.final_norm, d)
        self.head = build_part("head", spec.head, d)
        self._head_takes_out = "out" in inspect.signature(self.head.forward).parameters
        self.dtype: torch.dtype | None = None
        self.device: torch.device | None = None

    def parts(self):
        return [self.embedding, *self.blocks, self.final_norm, self.head]

    def tensor_specs(self) -> list[TensorSpec]:
        seen: dict[str, TensorSpec] = {}
        for part in self.parts():
            for s in part.tensor_specs():
                if s.name in seen and seen[s.name] != s:
                    raise ValueError(f"tensor {s.name} is declared twice with different shapes")
                seen[s.name] = s
        return list(seen.values())

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for part in self.parts():
            part.load(tensors)
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)
        self.dtype = self.embedding.table.dtype
        self.device = self.embedding.table.device

    def cache_requirements(self) -> list[tuple[PageSpec | None, list[StateSpec]]]:
        """For each entry of the run order: the pages and state it owns (none if it reads
        another entry's)."""
        out = []
        for call in self.schedule:
            mixer = self.blocks[call.layer].mixer
            if call.cache_from is not None:
                out.append((None, []))
            else:
                out.append((mixer.cache_spec(), mixer.state_specs()))
        return out

    def forward(self, ctx: StepContext, views: list[CacheView | None], logits_out: torch.Tensor | None = None) -> torch.Tensor:
        """Run the T tokens of the step; float32 logits [len(ctx.logits_rows), vocab], written
        into `logits_out` where the caller brings the buffer (a head whose `forward` takes no
        `out` has its result copied there)."""
        x = self.embedding.forward(ctx.token_ids)
        normed = None  # the next block's first norm of x, where the block before it has computed it
        for i, call in enumerate(self.schedule):
            own = call.cache_from is None
            then = self.blocks[self.schedule[i + 1].layer].mixer_norm if i + 1 < len(self.schedule) else None
            x, normed = self.blocks[call.layer].forward_chain(
                x, normed, ctx, views[i if own else call.cache_from], own, then
            )
        if ctx.logits_rows.shape[0] == 0:
            return torch.empty(0, self.spec.vocab_size, device=x.device, dtype=torch.float32)
        hidden = self.final_norm.forward(x, ctx.logits_rows)
        if logits_out is None:
            return self.head.forward(hidden)
        if self._head_takes_out:
            return self.head.forward(hidden, out=logits_out)
        return logits_out.copy_(self.head.forward(hidden))


def build_model(spec: ModelSpec) -> DecoderModel:
    return DecoderModel(spec)
