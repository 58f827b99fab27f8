"""One registry from an architecture's name (config.json `architectures[0]`) to its
configuration class and to the function that turns a configuration into a model
description (a `ModelSpec`: which parts, in which order, with which tensor names).

The reference knows one constant name (atomserve/config.py:11); here the same check is a
lookup, so that adding an architecture is one `register_architecture` call.
"""

from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Callable

from atomserve_b200.config.model_config import ModelConfigError


@dataclass(frozen=True)
class Architecture:
    name: str
    config_class: Any  # has from_dict(raw) and to_dict()
    build_spec: Callable[[Any], Any]  # config -> parts.spec.ModelSpec


_ARCHITECTURES: dict[str, Architecture] = {}


def register_architecture(name: str, config_class: Any, build_spec: Callable[[Any], Any]) -> None:
    _ARCHITECTURES[name] = Architecture(name, config_class, build_spec)


def architecture_for(name: str) -> Architecture:
    _ensure_builtin()
    if name not in _ARCHITECTURES:
        raise ModelConfigError(
            f"architecture {name!r} is not registered; known: {sorted(_ARCHITECTURES)}"
        )
    return _ARCHITECTURES[name]


def load_model_config(model_dir: str | Path) -> tuple[Architecture, Any]:
    """Read `<model_dir>/config.json` and parse it with the class its architecture names."""
    path = Path(model_dir) / "config.json"
    if not path.exists():
        raise FileNotFoundError(f"no config.json in {model_dir}")
    return config_from_dict(json.loads(path.read_text()))


def config_from_dict(raw: dict) -> tuple[Architecture, Any]:
    names = raw.get("architectures") or []
    if len(names) != 1:
        raise ModelConfigError(f"config.json must name exactly one architecture, got {names}")
    arch = architecture_for(names[0])
    return arch, arch.config_class.from_dict(raw)


def _ensure_builtin() -> None:
    if "Qwen3ForCausalLM" not in _ARCHITECTURES:
        from atomserve_b200.models import qwen3  # noqa: F401  (registers itself)
