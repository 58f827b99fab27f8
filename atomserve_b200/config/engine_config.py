"""Serving limits: how much cache exists and how much work one step may do.

Fields and checks follow the reference's EngineConfig (atomserve/config.py:68-92) without its
speculative-decoding and int8-cache fields.
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class EngineConfig:
    block_size: int = 16  # tokens per cache page
    num_blocks: int = 1024  # pages in each cache group's pool
    max_num_seqs: int = 32  # most requests running (holding pages and a state slot) at once
    max_num_batched_tokens: int = 512  # token budget of one step
    max_model_len: int = 16384  # longest sequence (prompt + output) accepted
    enable_prefix_caching: bool = True  # share pages of identical prompt prefixes
    cuda_graphs: bool = True  # replay captured graphs for decode-only steps
    decode_lookahead: bool = True  # launch a decode-only step before the one before it has been read

    def __post_init__(self) -> None:
        if self.block_size < 1 or self.num_blocks < 1 or self.max_num_seqs < 1:
            raise ValueError("block_size, num_blocks and max_num_seqs must be positive")
        if self.max_model_len > self.num_blocks * self.block_size:
            # Otherwise a lone sequence could outgrow the pool with nobody left to preempt.
            raise ValueError(
                f"max_model_len {self.max_model_len} exceeds the cache pool's "
                f"{self.num_blocks * self.block_size} tokens"
            )
        if self.max_num_batched_tokens < self.max_num_seqs:
            raise ValueError("max_num_batched_tokens must be >= max_num_seqs (one decode each)")
