"""Weights from safetensors files, fetched by tensor name.

The model says which tensors it needs (name, shape, kind); the files are checked against that
list before anything is read, and one error names everything that is wrong: tensors missing,
tensors nobody asked for, and shapes that differ. Matrices are cast to the compute dtype
(bfloat16 when serving), gains stay float32, integer tables become int32. Tensors are read one
at a time and moved to the device, so the host never holds the checkpoint whole
(atomserve/loader.py:63-148 is the reference's loader: same names, no shape check).
"""

from __future__ import annotations

import json
from contextlib import ExitStack
from pathlib import Path
from typing import Any

import torch
from safetensors import safe_open

from atomserve_b200.config.registry import Architecture, load_model_config
from atomserve_b200.parts.model import DecoderModel, build_model
from atomserve_b200.parts.spec import TensorSpec

COMPUTE_DTYPES = {
    "bfloat16": torch.bfloat16, "bf16": torch.bfloat16,
    "float32": torch.float32, "fp32": torch.float32,
}  # fmt: skip


class WeightsError(ValueError):
    """The checkpoint does not hold what the model needs."""


def final_dtype(spec: TensorSpec, compute_dtype: torch.dtype) -> torch.dtype:
    if spec.kind == "matrix":
        return compute_dtype
    if spec.kind == "gain":
        return torch.float32
    if spec.kind == "int":
        return torch.int32
    raise ValueError(f"tensor {spec.name} has unknown kind {spec.kind!r}")


class _FileTensors:
    """Lazy mapping name -> tensor on the device, in its final dtype."""

    def __init__(self, where: dict[str, Any], specs: dict[str, TensorSpec], dtype: torch.dtype, device: torch.device):
        self.where, self.specs, self.dtype, self.device = where, specs, dtype, device

    def __getitem__(self, name: str) -> torch.Tensor:
        t = self.where[name].get_tensor(name)
        return t.to(device=self.device, dtype=final_dtype(self.specs[name], self.dtype))


def check_names_and_shapes(found: dict[str, tuple[int, ...]], specs: list[TensorSpec], ignored: tuple[str, ...],
                           duplicated: dict[str, list[str]] | None = None) -> None:  # fmt: skip
    """One error for everything that is wrong with a checkpoint: names the model needs and the
    files lack, names the files hold and the model does not know, shapes that differ, and names
    that more than one file of the folder holds (`duplicated`: name -> those files)."""
    wanted = {s.name: s for s in specs}
    missing = sorted(n for n in wanted if n not in found)
    unexpected = sorted(n for n in found if n not in wanted and n not in ignored)
    wrong = sorted(
        f"{n}: file has {list(found[n])}, model needs {list(s.shape)}"
        for n, s in wanted.items()
        if n in found and tuple(found[n]) != tuple(s.shape)
    )
    twice = sorted(f"{n} (in {', '.join(files)})" for n, files in (duplicated or {}).items())
    if missing or unexpected or wrong or twice:
        lines = ["checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing tensors ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected tensors ({len(unexpected)}): " + ", ".join(unexpected))
        if wrong:
            lines.append(f"  wrong shapes ({len(wrong)}): " + "; ".join(wrong))
        if twice:
            lines.append(f"  tensors held by more than one file ({len(twice)}): " + "; ".join(twice))
        raise WeightsError("\n".join(lines))


def checkpoint_files(model_dir: Path) -> list[Path]:
    """The safetensors files that make up the folder's checkpoint: those that
    `model.safetensors.index.json` names where the folder has that index (other files lying
    about are then not part of the model), else every `*.safetensors` file."""
    index = model_dir / "model.safetensors.index.json"
    if index.exists():
        named = sorted(set(json.loads(index.read_text()).get("weight_map", {}).values()))
        absent = [n for n in named if not (model_dir / n).exists()]
        if absent:
            raise FileNotFoundError(f"{index.name} names files that {model_dir} lacks: {', '.join(absent)}")
        if named:
            return [model_dir / n for n in named]
    return sorted(model_dir.glob("*.safetensors"))


def load_tensors_into(model: DecoderModel, model_dir: str | Path, dtype: torch.dtype, device: torch.device | str) -> None:
    """Check the folder's safetensors files against the model, then load them."""
    shards = checkpoint_files(Path(model_dir))
    if not shards:
        raise FileNotFoundError(f"no *.safetensors files in {model_dir}")
    specs = model.tensor_specs()
    with ExitStack() as stack:
        files = [stack.enter_context(safe_open(str(s), framework="pt", device="cpu")) for s in shards]
        where: dict[str, Any] = {}
        holders: dict[str, list[str]] = {}
        for shard, f in zip(shards, files):
            for name in f.keys():  # noqa: SIM118
                where.setdefault(name, f)
                holders.setdefault(name, []).append(shard.name)
        found = {name: tuple(f.get_slice(name).get_shape()) for name, f in where.items()}
        duplicated = {n: fs for n, fs in holders.items() if len(fs) > 1}
        check_names_and_shapes(found, specs, model.spec.ignored_tensors, duplicated)
        model.load(_FileTensors(where, {s.name: s for s in specs}, dtype, torch.device(device)))


def load_model(model_dir: str | Path, dtype: str | torch.dtype = "bfloat16", device: torch.device | str = "cuda"):
    """config.json -> architecture -> model, with the folder's weights. Returns (arch, config, model)."""
    arch, config = load_model_config(model_dir)
    model = build_model(arch.build_spec(config))
    load_tensors_into(model, model_dir, parse_dtype(dtype), device)
    return arch, config, model


def parse_dtype(dtype: str | torch.dtype) -> torch.dtype:
    if isinstance(dtype, torch.dtype):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError(f"compute dtype must be bfloat16 or float32, got {dtype}")
        return dtype
    try:
        return COMPUTE_DTYPES[dtype]
    except KeyError:
        raise ValueError(f"unknown dtype {dtype!r}; choose from {sorted(COMPUTE_DTYPES)}") from None


def read_eos_token_ids(model_dir: str | Path) -> frozenset[int]:
    """End-of-sequence ids from generation_config.json (`eos_token_id`: int or list), else none
    (atomserve/tokenizer.py:36-38 reads the same key)."""
    path = Path(model_dir) / "generation_config.json"
    if not path.exists():
        return frozenset()
    eos = json.loads(path.read_text()).get("eos_token_id")
    if eos is None:
        return frozenset()
    return frozenset(eos if isinstance(eos, list) else [eos])


__all__ = ["Architecture", "WeightsError", "load_model", "load_tensors_into", "parse_dtype", "read_eos_token_ids"]
