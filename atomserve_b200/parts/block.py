"""The pre-norm residual arrangement: x = x + mixer(norm(x)); x = x + ff(norm(x))
(atomserve/model.py:11-13, 378-382). The residual additions happen inside the mixer's and the
feed-forward's last projection, so the block only routes tensors."""

from __future__ import annotations

import torch

from atomserve_b200.parts.base import Block, CacheView, Norm, StepContext, register_part


class PreNormBlock(Block):
    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        return self.forward_chain(x, None, ctx, cache, write_cache, None)[0]

    def forward_chain(self, x: torch.Tensor, normed: torch.Tensor | None, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
        # each projection that ends a part is handed the norm that follows it, so that the part
        # may fuse the two (the norm after the feed-forward belongs to the next block)
        if normed is None:
            normed = self.mixer_norm.forward(x)
        x, normed = self.mixer.forward_then(normed, x, ctx, cache, write_cache, self.feed_forward_norm)
        if then is None:
            return self.feed_forward.forward(normed, x, ctx), None
        return self.feed_forward.forward_then(normed, x, ctx, then)


register_part("block", "pre_norm", PreNormBlock)
