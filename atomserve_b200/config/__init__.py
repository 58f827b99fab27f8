from atomserve_b200.config.engine_config import EngineConfig
from atomserve_b200.config.model_config import ModelConfigError, Qwen3Config
from atomserve_b200.config.registry import (
    Architecture,
    architecture_for,
    load_model_config,
    register_architecture,
)

__all__ = [
    "Architecture",
    "EngineConfig",
    "ModelConfigError",
    "Qwen3Config",
    "architecture_for",
    "load_model_config",
    "register_architecture",
]
