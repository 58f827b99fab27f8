"""Token embedding (a gather, no scaling, atomserve/model.py:373) and the output head
(float32 logits from the float32 accumulator, atomserve/model.py:388-412; tied to the
embedding when the model says so, atomserve/loader.py:131-138)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import Part, register_part
from atomserve_b200.parts.spec import TensorSpec


class TokenEmbedding(Part):
    def __init__(self, hidden_size: int, prefix: str, vocab_size: int):
        self.hidden_size, self.vocab_size, self.name = hidden_size, vocab_size, prefix + "weight"
        self.table: torch.Tensor | None = None
        self.status: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.table = tensors[self.name]
        # the device's shared status words on a GPU (the engine reads them every step)
        self.status = (ops.status_for(self.table.device).embedding if self.table.is_cuda
                       else torch.zeros(1, dtype=torch.int32))

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return ops.embedding(token_ids, self.table, self.status)


class LMHead(Part):
    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, tied: bool):
        self.hidden_size, self.vocab_size, self.tied, self.name = hidden_size, vocab_size, tied, prefix + "weight"
        self.weight: torch.Tensor | None = None

    def tensor_specs(self) -> list[TensorSpec]:
        return [] if self.tied else [TensorSpec(self.name, (self.vocab_size, self.hidden_size))]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = tensors[self.name]

    def tie(self, embedding: TokenEmbedding) -> None:
        self.weight = embedding.table

    def forward(self, hidden: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
        return ops.linear(hidden, self.weight, out_dtype=torch.float32, out=out)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
