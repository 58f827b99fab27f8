"""Dense SwiGLU feed-forward: residual + down( silu(gate(h)) * up(h) ), no biases
(atomserve/model.py:339-360)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import FeedForward, Norm, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class SwiGLU(FeedForward):
    def __init__(self, hidden_size: int, prefix: str, intermediate_size: int):
        self.hidden_size, self.prefix, self.intermediate_size = hidden_size, prefix, intermediate_size
        self.gate_up_proj = self.down_proj = None
        self.fused = False

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, i = self.prefix, self.hidden_size, self.intermediate_size
        return [
            TensorSpec(p + "gate_proj.weight", (i, d)),
            TensorSpec(p + "up_proj.weight", (i, d)),
            TensorSpec(p + "down_proj.weight", (d, i)),
        ]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        gate, up = tensors[p + "gate_proj.weight"], tensors[p + "up_proj.weight"]
        self.fused = gate.is_cuda and ops.swiglu_fusable(gate)
        if self.fused:
            # rows alternate gate_i, up_i: the tensor-core GEMM applies SiLU * up in its epilogue
            self.gate_up_proj = ops.interleave_gate_up(gate, up)
        else:
            # gate rows first, then up rows (atomserve/loader.py:121)
            self.gate_up_proj = torch.cat([gate, up]).contiguous()
        self.down_proj = tensors[p + "down_proj.weight"]

    def hidden(self, h: torch.Tensor) -> torch.Tensor:
        if self.fused:
            return ops.linear_swiglu(h, self.gate_up_proj)
        return ops.silu_mul(ops.linear(h, self.gate_up_proj))

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ops.linear(self.hidden(h), self.down_proj, residual)

    def forward_then(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext,
                     then: Norm) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        after_linear = getattr(then, "after_linear", None)
        if after_linear is None:
            return super().forward_then(h, residual, ctx, then)
        return after_linear(self.hidden(h), self.down_proj, residual)


register_part("feed_forward", "swiglu", SwiGLU)
