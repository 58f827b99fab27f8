"""The pre-norm residual arrangement: x = x + mixer(norm(x)); x = x + ff(norm(x))
(atomserve/model.py:11-13, 378-382). The residual additions happen inside the mixer's and the
feed-forward's last projection, so the block only routes tensors."""

from __future__ import annotations

import torch

from atomserve_b200.parts.base import Block, CacheView, StepContext, register_part


class PreNormBlock(Block):
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        x = self.mixer.forward(self.mixer_norm.forward(x), x, ctx, cache, write_cache)
        return self.feed_forward.forward(self.feed_forward_norm.forward(x), x, ctx)


register_part("block", "pre_norm", PreNormBlock)
