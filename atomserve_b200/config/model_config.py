"""Typed model configuration, read from the architecture's own config.json keys.

Every size and constant the model computes with comes from here; none is written into
the parts or the kernels. The keys, defaults and rejections follow the reference's
ModelConfig (atomserve/config.py:15-65). Two things go beyond it and are stated as such:
divisibility checks that the reference leaves to a later shape error, and the sliding
window, which the reference rejects (atomserve/config.py:43-44) and this engine runs.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path


class ModelConfigError(ValueError):
    """config.json describes a model this engine does not run."""


@dataclass(frozen=True)
class Qwen3Config:
    """Shape and numerics of a Qwen3 dense decoder (`Qwen3ForCausalLM`)."""

    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    # Layers with index >= max_window_layers attend to the last `sliding_window` positions
    # (self included) when use_sliding_window is set; otherwise every layer sees all keys.
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int = 0

    architecture = "Qwen3ForCausalLM"

    @classmethod
    def from_dict(cls, raw: dict) -> "Qwen3Config":
        """Build from a parsed config.json; fail fast on what would change the math."""
        architectures = raw.get("architectures") or []
        if architectures != [cls.architecture]:
            raise ModelConfigError(f"expected architectures [{cls.architecture!r}], got {architectures}")
        if raw.get("attention_bias"):
            raise ModelConfigError("attention_bias=True is not supported")
        if raw.get("rope_scaling"):
            raise ModelConfigError("rope_scaling is not supported")
        if raw.get("hidden_act", "silu") != "silu":
            raise ModelConfigError(f"hidden_act={raw['hidden_act']} is not supported")
        missing = [
            k
            for k in (
                "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                "num_attention_heads", "num_key_value_heads", "rms_norm_eps", "rope_theta",
                "max_position_embeddings",
            )  # fmt: skip
            if k not in raw
        ]
        if missing:
            raise ModelConfigError(f"config.json lacks required keys: {missing}")
        use_window = bool(raw.get("use_sliding_window", False))
        config = cls(
            vocab_size=int(raw["vocab_size"]),
            hidden_size=int(raw["hidden_size"]),
            intermediate_size=int(raw["intermediate_size"]),
            num_hidden_layers=int(raw["num_hidden_layers"]),
            num_attention_heads=int(raw["num_attention_heads"]),
            num_key_value_heads=int(raw["num_key_value_heads"]),
            head_dim=int(raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"]),
            rms_norm_eps=float(raw["rms_norm_eps"]),
            rope_theta=float(raw["rope_theta"]),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            max_position_embeddings=int(raw["max_position_embeddings"]),
            use_sliding_window=use_window,
            sliding_window=int(raw["sliding_window"]) if use_window else None,
            max_window_layers=int(raw.get("max_window_layers", 0)) if use_window else 0,
        )
        config.validate()
        return config

    def validate(self) -> None:
        for name in (
            "vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
            "num_attention_heads", "num_key_value_heads", "head_dim", "max_position_embeddings",
        ):  # fmt: skip
            if getattr(self, name) < 1:
                raise ModelConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ModelConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ModelConfigError(f"head_dim {self.head_dim} must be even for rotary pairs")
        if not self.rms_norm_eps >= 0 or not self.rope_theta > 0:
            raise ModelConfigError("rms_norm_eps must be >= 0 and rope_theta > 0")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window < 1):
            raise ModelConfigError("use_sliding_window needs a positive sliding_window")

    def window_of_layer(self, layer: int) -> int | None:
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        raw = {
            "architectures": [self.architecture],
            "model_type": "qwen3",
            "vocab_size": self.vocab_size,
            "hidden_size": self.hidden_size,
            "intermediate_size": self.intermediate_size,
            "num_hidden_layers": self.num_hidden_layers,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "hidden_act": "silu",
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": False,
            "use_sliding_window": self.use_sliding_window,
        }
        if self.use_sliding_window:
            raw["sliding_window"] = self.sliding_window
            raw["max_window_layers"] = self.max_window_layers
        return raw

    @classmethod
    def load(cls, model_dir: Path) -> "Qwen3Config":
        return cls.from_dict(json.loads((Path(model_dir) / "config.json").read_text()))
