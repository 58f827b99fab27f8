"""Seeded random weights: for a model in memory, or written out as a model folder
(config.json + model.safetensors) that the ordinary loader then reads.

Matrices are N(0, 0.02), norm gains 1 + N(0, 0.1). Every tensor has its own generator seeded
from (seed, tensor name), so a tensor's values do not depend on which other tensors exist or
in which order they are made. (The reference has random weights only in its tests,
tests/conftest.py:45-70.)
"""

from __future__ import annotations

import hashlib
import json
from pathlib import Path
from typing import Any

import torch
from safetensors.torch import save_file

from atomserve_b200.config.registry import architecture_for
from atomserve_b200.parts.model import DecoderModel, build_model
from atomserve_b200.parts.spec import TensorSpec
from atomserve_b200.weights.loader import final_dtype, parse_dtype


def _seed_for(seed: int, name: str) -> int:
    digest = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(digest[:8], "little") & 0x7FFFFFFFFFFFFFFF


def random_tensor(spec: TensorSpec, seed: int, dtype: torch.dtype, device: torch.device) -> torch.Tensor:
    g = torch.Generator(device=device)
    g.manual_seed(_seed_for(seed, spec.name))
    if spec.init == "normal":
        t = torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * 0.02
    elif spec.init == "gain":
        t = 1.0 + torch.randn(spec.shape, generator=g, device=device, dtype=torch.float32) * 0.1
    elif spec.init == "zeros":
        t = torch.zeros(spec.shape, device=device, dtype=torch.float32)
    elif spec.init == "index":
        t = torch.randint(0, max(spec.high, 1), spec.shape, generator=g, device=device)
    else:
        raise ValueError(f"tensor {spec.name} has unknown init {spec.init!r}")
    return t.to(dtype)


class RandomTensors:
    """Lazy mapping name -> seeded random tensor, made on `device` in its final dtype."""

    def __init__(self, specs: list[TensorSpec], seed: int, dtype: torch.dtype, device: torch.device | str):
        self.specs = {s.name: s for s in specs}
        self.seed, self.dtype, self.device = seed, dtype, torch.device(device)

    def __getitem__(self, name: str) -> torch.Tensor:
        spec = self.specs[name]
        return random_tensor(spec, self.seed, final_dtype(spec, self.dtype), self.device)


def random_model(config: Any, seed: int, dtype: str | torch.dtype = "bfloat16", device: torch.device | str = "cuda") -> DecoderModel:
    """A model of `config`'s architecture with random weights made directly on the device."""
    arch = architecture_for(config.architecture)
    model = build_model(arch.build_spec(config))
    model.load(RandomTensors(model.tensor_specs(), seed, parse_dtype(dtype), device))
    return model


def write_model_folder(config: Any, seed: int, out_dir: str | Path, dtype: str | torch.dtype = "bfloat16",
                       eos_token_ids: list[int] | None = None) -> Path:  # fmt: skip
    """Write config.json and model.safetensors for `config` with weights drawn from `seed`.
    Matrices are stored in `dtype`; gains in float32."""
    out = Path(out_dir)
    out.mkdir(parents=True, exist_ok=True)
    arch = architecture_for(config.architecture)
    model = build_model(arch.build_spec(config))
    store = parse_dtype(dtype)
    tensors = {
        s.name: random_tensor(s, seed, final_dtype(s, store), torch.device("cpu")).contiguous()
        for s in model.tensor_specs()
    }
    (out / "config.json").write_text(json.dumps(config.to_dict(), indent=2) + "\n")
    if eos_token_ids is not None:
        (out / "generation_config.json").write_text(json.dumps({"eos_token_id": eos_token_ids}) + "\n")
    save_file(tensors, str(out / "model.safetensors"), metadata={"format": "pt"})
    return out
