"""Descriptions of a model as data: which parts, with which sizes, under which tensor names,
run in which order. An architecture's `build_spec(config)` returns a `ModelSpec`; everything
below it (loader, random weights, model builder, cache manager, step function) works from the
spec alone and does not know the architecture's name.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class TensorSpec:
    """One checkpoint tensor a part needs.

    kind: "matrix"  stored in the compute dtype (bfloat16 when serving, float32 on the 32-bit path)
          "gain"    a norm gain or other small vector; kept in float32 whatever it is stored as
          "int"     an integer table; kept as int32
    init: how the random-weights mode fills it: "normal" N(0, 0.02), "gain" 1 + N(0, 0.1),
          "zeros", or "index" (integers below `high`).
    """

    name: str
    shape: tuple[int, ...]
    kind: str = "matrix"
    init: str = "normal"
    high: int = 0


@dataclass(frozen=True)
class PartSpec:
    """A part by kind (its name in the part registry), its parameters, and the prefix its
    tensor names hang under in the checkpoint."""

    kind: str
    params: dict[str, Any] = field(default_factory=dict)
    prefix: str = ""


@dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement over a mixer and a feed-forward with their norms."""

    block: str  # kind in the block registry, e.g. "pre_norm"
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order. `layer` indexes ModelSpec.layers (the same layer may be
    called twice: shared weights, separate caches). `cache_from`, if set, is the index of an
    earlier entry of the run order whose cache this call reads instead of owning one."""

    layer: int
    cache_from: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    max_positions: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    schedule: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    # checkpoint names that may be present and are ignored (a tied model shipping a head copy)
    ignored_tensors: tuple[str, ...] = ()
