"""Interfaces of the parts a model is assembled from, their registries, and the per-step
context they compute in.

A part is built from its `PartSpec` parameters and the model's hidden size; it names the
checkpoint tensors it needs, receives them once, and computes on the flat batch. No part
knows which model it is in or which layer it is.

  Norm            forward(x, rows=None) -> same width
  PositionEncoding  how positions enter a mixer: fused_rotary() or encode(q, k, ctx)
  Mixer           forward(h, residual, ctx, cache, write_cache) -> residual + mix(h);
                  cache_spec() says what it keeps in pages between steps (keys and values, or
                  any other tensors per token), state_specs() what it keeps at fixed size
  FeedForward     forward(h, residual, ctx) -> residual + ff(h)
  Block           arranges a mixer and a feed-forward with their norms around the residual
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Callable

import torch

from atomserve_b200.parts.spec import PartSpec, TensorSpec


# ---- what a mixer keeps between steps -------------------------------------------------------


@dataclass(frozen=True)
class PageTensor:
    """One of the tensors a cache page holds: per token, `heads` vectors of `width` values. The
    pool of it is [entries, num_blocks, heads, block_size, width] in the cache dtype."""

    name: str
    heads: int
    width: int


@dataclass(frozen=True)
class PageSpec:
    """What a mixer keeps in pages: the tensors each page holds, and `window`: only the last
    `window` positions are ever read, so older pages can be given back early. Entries of the run
    order with equal specs share a group of pools, an allocator and the requests' block tables."""

    tensors: tuple[PageTensor, ...]
    window: int | None = None

    @property
    def values_per_token(self) -> int:
        return sum(t.heads * t.width for t in self.tensors)


def KVCacheSpec(num_kv_heads: int, head_dim: int, window: int | None = None) -> PageSpec:
    """The usual pages: keys and values, `num_kv_heads * head_dim` of each per token, as tensors
    "k" and "v"."""
    return PageSpec((PageTensor("k", num_kv_heads, head_dim), PageTensor("v", num_kv_heads, head_dim)), window)


@dataclass(frozen=True)
class StateSpec:
    """Fixed-size per-request state: one tensor of `shape` per request slot, zero at admission."""

    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype = torch.float32


class CacheView:
    """What one entry of the run order sees of the cache during a step.

    `pages[name]` is [num_blocks, heads, block_size, width] for each tensor of the entry's
    PageSpec (`k` and `v` are shorthands for the pages of those names); `slots` [T] int32 says
    where each new token is written; `block_tables` [R, W] int32 where each request's positions
    live. For state: `state[name]` is [num_slots, *shape], indexed by ctx.state_slots.
    """

    def __init__(self, k: torch.Tensor | None = None, v: torch.Tensor | None = None, slots: torch.Tensor | None = None,
                 block_tables: torch.Tensor | None = None, block_size: int = 0,
                 state: dict[str, torch.Tensor] | None = None, pages: dict[str, torch.Tensor] | None = None):  # fmt: skip
        self.pages: dict[str, torch.Tensor] = dict(pages or {})
        if k is not None:
            self.pages["k"] = k
        if v is not None:
            self.pages["v"] = v
        self.slots, self.block_tables, self.block_size = slots, block_tables, block_size
        self.state: dict[str, torch.Tensor] = state if state is not None else {}

    @property
    def k(self) -> torch.Tensor | None:
        return self.pages.get("k")

    @k.setter
    def k(self, pages: torch.Tensor) -> None:
        self.pages["k"] = pages

    @property
    def v(self) -> torch.Tensor | None:
        return self.pages.get("v")

    @v.setter
    def v(self, pages: torch.Tensor) -> None:
        self.pages["v"] = pages


# ---- the step's batch as parts see it -------------------------------------------------------


@dataclass
class StepContext:
    """One step's flat batch: T new tokens of R requests, each request's tokens contiguous.

    Device tensors are int32. Host copies (`host_*`) are for parts that plan on the host.
    """

    num_tokens: int
    num_requests: int
    token_ids: torch.Tensor  # [T]
    positions: torch.Tensor  # [T] absolute position of each token in its request
    req_q_start: torch.Tensor  # [R + 1] first row of each request
    req_pos_start: torch.Tensor  # [R] position of each request's first new token
    state_slots: torch.Tensor  # [R] per-request state slot
    logits_rows: torch.Tensor  # [B'] rows whose logits are wanted
    max_context: int  # largest position + 1 reached by any request in this step
    host_q_lens: list[int] = field(default_factory=list)
    host_pos_start: list[int] = field(default_factory=list)
    host_state_slots: list[int] = field(default_factory=list)


# ---- interfaces -----------------------------------------------------------------------------


class Part:
    """Common to all parts: the tensors it needs and how it takes them."""

    def tensor_specs(self) -> list[TensorSpec]:
        return []

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        """Receive the tensors named by tensor_specs (on the device, in their final dtype)."""


class Norm(Part):
    def forward(self, x: torch.Tensor, rows: torch.Tensor | None = None) -> torch.Tensor:
        raise NotImplementedError

    # A norm may also offer `after_linear(x, weight, residual) -> (s, forward(s))` with
    # s = x . weight^T + residual: a mixer or feed-forward whose last step is such a projection
    # hands it to the norm that follows, which may then run both in one kernel.


@dataclass(frozen=True)
class FusedRotary:
    """An encoding that a mixer's fused kernel can apply by itself: each head's first
    `rotary_dim` dimensions are turned, pair (i, i + rotary_dim / 2) by the angle
    position * inv_freq[i] (`inv_freq`: float32 [rotary_dim / 2] on the device)."""

    inv_freq: torch.Tensor
    rotary_dim: int


class PositionEncoding(Part):
    """How positions enter a mixer. The encoding owns how it is applied; a mixer asks it, in
    this order:

      fused_rotary()      a `FusedRotary` if the encoding is a rotation by position * frequency:
                          the mixer's fused kernel then applies it on the way to the cache;
      encode(q, k, ctx)   otherwise: the queries [T, H, hd] and keys [T, KV, hd] (after their
                          norm, before the keys are stored) with the positions of the step's
                          tokens worked in, by whatever rule. The default changes nothing (an
                          encoding that acts elsewhere, or none).

    `prepare(device)` builds its tables once."""

    def prepare(self, device: torch.device) -> None:
        pass

    def fused_rotary(self) -> FusedRotary | None:
        # encodings written against the older convention carry the two fields themselves
        inv_freq, rotary_dim = getattr(self, "inv_freq", None), getattr(self, "rotary_dim", None)
        if inv_freq is not None and rotary_dim:
            return FusedRotary(inv_freq, rotary_dim)
        return None

    def encode(self, q: torch.Tensor, k: torch.Tensor | None, ctx: "StepContext") -> tuple[torch.Tensor, torch.Tensor | None]:
        return q, k


class Mixer(Part):
    def cache_spec(self) -> PageSpec | None:
        """The pages this mixer keeps (`KVCacheSpec(...)` for keys and values; any other list of
        tensors as a `PageSpec`), or None."""
        return None

    def state_specs(self) -> list[StateSpec]:
        return []

    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        raise NotImplementedError

    def forward_then(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                     write_cache: bool, then: Norm) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        """(out, then(out)) for out = forward(...): the block calls this when a norm follows, so
        that a mixer can fuse its last projection with that norm. The default runs them in turn."""
        out = self.forward(h, residual, ctx, cache, write_cache)
        return out, then.forward(out)


class FeedForward(Part):
    def forward(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError

    def forward_then(self, h: torch.Tensor, residual: torch.Tensor, ctx: StepContext,
                     then: Norm) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
        """(out, then(out)) for out = forward(...); see Mixer.forward_then."""
        out = self.forward(h, residual, ctx)
        return out, then.forward(out)


class Block(Part):
    def __init__(self, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm):
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm

    def parts(self) -> list[Part]:
        return [self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward]

    def tensor_specs(self) -> list[TensorSpec]:
        return [s for p in self.parts() for s in p.tensor_specs()]

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        for p in self.parts():
            p.load(tensors)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView | None,
                write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        raise NotImplementedError

    def forward_chain(self, x: torch.Tensor, normed: torch.Tensor | None, ctx: StepContext, cache: CacheView | None,
                      write_cache: bool, then: Norm | None) -> tuple[torch.Tensor, torch.Tensor | None]:  # fmt: skip
        """forward() for a block inside a run of blocks, which is how the model calls it. `normed`
        is mixer_norm(x) where the previous block has computed it already; `then` is the norm
        that the next block applies first. Returns (result, then(result)), or (result, None)
        where the block leaves that norm to the next one, as this default does."""
        return self.forward(x, ctx, cache, write_cache), None


# ---- registries ------------------------------------------------------------------------------

_REGISTRIES: dict[str, dict[str, Callable[..., Any]]] = {
    "norm": {}, "position": {}, "mixer": {}, "feed_forward": {}, "block": {}, "embedding": {}, "head": {},
}  # fmt: skip


def register_part(family: str, kind: str, factory: Callable[..., Any]) -> None:
    """Make `kind` buildable. `factory(hidden_size=..., prefix=..., **params)` returns the part
    (a block's factory takes the four built parts instead)."""
    if family not in _REGISTRIES:
        raise KeyError(f"unknown part family {family!r}; families: {sorted(_REGISTRIES)}")
    _REGISTRIES[family][kind] = factory


def build_part(family: str, spec: PartSpec, hidden_size: int) -> Any:
    _ensure_builtin()
    try:
        factory = _REGISTRIES[family][spec.kind]
    except KeyError:
        raise KeyError(f"no {family} part of kind {spec.kind!r}; known: {sorted(_REGISTRIES[family])}") from None
    return factory(hidden_size=hidden_size, prefix=spec.prefix, **spec.params)


def build_block(kind: str, mixer: Mixer, feed_forward: FeedForward, mixer_norm: Norm, feed_forward_norm: Norm) -> Block:
    _ensure_builtin()
    try:
        factory = _REGISTRIES["block"][kind]
    except KeyError:
        raise KeyError(f"no block of kind {kind!r}; known: {sorted(_REGISTRIES['block'])}") from None
    return factory(mixer, feed_forward, mixer_norm, feed_forward_norm)


def _ensure_builtin() -> None:
    if "rms_norm" not in _REGISTRIES["norm"]:
        from atomserve_b200.parts import attention, block, embedding, mlp, norms, rotary  # noqa: F401
