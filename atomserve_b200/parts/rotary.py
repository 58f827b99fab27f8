"""Rotary position encoding: pair i of rotary_dim/2 turns by position * theta^(-2i/rotary_dim),
rotate-half pairing (i, i + rotary_dim/2); angles in float32 (atomserve/model.py:142-185).
Dimensions beyond rotary_dim pass through unrotated (rotary_dim = head_dim for Qwen3)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import FusedRotary, PositionEncoding, register_part


class Rotary(PositionEncoding):
    def __init__(self, hidden_size: int, prefix: str, head_dim: int, theta: float, rotary_dim: int | None = None):
        self.head_dim = head_dim
        self.rotary_dim = rotary_dim or head_dim
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        self.inv_freq: torch.Tensor | None = None

    def prepare(self, device: torch.device) -> None:
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta**exponents)).to(device)

    def fused_rotary(self) -> FusedRotary:
        return FusedRotary(self.inv_freq, self.rotary_dim)

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotate x [T, heads, head_dim] by its tokens' positions (the encoding on its own)."""
        return ops.rotary(x, positions, self.inv_freq, self.rotary_dim)


register_part("position", "rotary", Rotary)
