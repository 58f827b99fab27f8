"""RMSNorm: gain * x / sqrt(mean(x^2) + eps), float32 inside, one rounding
(atomserve/model.py:125-139)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import Norm, register_part
from atomserve_b200.parts.spec import TensorSpec


class RMSNorm(Norm):
    def __init__(self, hidden_size: int, prefix: str, eps: float, width: int | None = None):
        self.width = width or hidden_size
        self.eps = float(eps)
        self.name = prefix + "weight"
        self.gain: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.width,), kind="gain", init="gain")]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.gain = tensors[self.name]

    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        return ops.rms_norm(x, self.gain, self.eps, rows)

    def after_linear(self, x: torch.Tensor, weight: torch.Tensor,
                     residual: torch.Tensor | None) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        """(s, forward(s)) for s = x . weight^T + residual. Where the product runs with partial
        sums (few tokens), one kernel adds them up, adds the residual and normalises; the results
        are the same bits either way."""
        if ops.partial_add_rms_norm_fusable(self.width) and weight.shape[0] == self.width:
            product = ops.linear_partial(x, weight)
            if product is not None:
                return ops.partial_add_rms_norm(product, residual, self.gain, self.eps)
        total = ops.linear(x, weight, residual)
        return total, self.forward(total)


register_part("norm", "rms_norm", RMSNorm)
