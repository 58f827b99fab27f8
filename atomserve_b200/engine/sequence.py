"""A sequence: one request's tokens, its sampling settings and what it holds of the cache.

    WAITING --admit--> RUNNING --end of sequence / max_tokens / abort--> FINISHED
       ^                  |
       +----preempt-------+   (pages and state slot given back; recomputed when readmitted)

The runner only reads sequences; the scheduler alone changes them, on the engine thread.
Fields and rules follow atomserve/sequence.py:17-115 (without the draft-model counters).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from enum import Enum

from atomserve_b200.cache.manager import RequestCache


class SequenceStatus(Enum):
    WAITING = "waiting"
    RUNNING = "running"
    FINISHED = "finished"


@dataclass(frozen=True)
class SamplingParams:
    """How to pick each next token, and when to stop (atomserve/sequence.py:23-43).

    temperature 0 is greedy; top_k 0 (or >= vocabulary) keeps all; top_p keeps the smallest
    set of most likely tokens whose mass reaches it; presence_penalty is subtracted once from
    the logit of every distinct token already generated; seed fixes the request's own random
    stream, independent of its batch neighbours.
    """

    temperature: float = 0.6
    top_k: int = 20
    top_p: float = 0.95
    presence_penalty: float = 0.0
    max_tokens: int = 4096
    seed: int | None = None
    ignore_eos: bool = False


THINKING_PARAMS = SamplingParams(temperature=0.6, top_p=0.95, top_k=20)
NON_THINKING_PARAMS = SamplingParams(temperature=0.7, top_p=0.8, top_k=20)


@dataclass(eq=False)
class Sequence:
    id: int
    token_ids: list[int]
    params: SamplingParams = field(default_factory=SamplingParams)
    num_prompt_tokens: int = -1
    num_computed_tokens: int = 0  # leading tokens whose keys and values are in the cache
    cache: RequestCache | None = None  # block tables per cache group and the state slot
    num_cached_tokens: int = 0  # prompt tokens found in the prefix cache at admission
    status: SequenceStatus = SequenceStatus.WAITING
    finish_reason: str | None = None  # "stop", "length" or "abort"

    def __post_init__(self) -> None:
        if self.num_prompt_tokens < 0:
            self.num_prompt_tokens = len(self.token_ids)

    @property
    def num_tokens(self) -> int:
        return len(self.token_ids)

    @property
    def output_ids(self) -> list[int]:
        return self.token_ids[self.num_prompt_tokens :]

    def reaches_end(self, num_new_tokens: int) -> bool:
        """Whether computing `num_new_tokens` more covers every known token: only then is
        there a next token to predict (atomserve/sequence.py:93-100)."""
        return self.num_computed_tokens + num_new_tokens == len(self.token_ids)


@dataclass
class StepResult:
    """What one step did for one scheduled sequence: the sampled tokens (none for a portion
    that stops short) and how many leading tokens are now in the cache."""

    tokens: list[int]
    num_computed: int
