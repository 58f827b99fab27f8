from atomserve_b200.parts.base import (
    Block,
    CacheView,
    FeedForward,
    FusedRotary,
    KVCacheSpec,
    Mixer,
    Norm,
    PageSpec,
    PageTensor,
    Part,
    PositionEncoding,
    StateSpec,
    StepContext,
    build_block,
    build_part,
    register_part,
)
from atomserve_b200.parts.model import DecoderModel, build_model
from atomserve_b200.parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec, TensorSpec

__all__ = [
    "Block", "CacheView", "DecoderModel", "FeedForward", "FusedRotary", "KVCacheSpec", "LayerCall", "LayerSpec",
    "Mixer", "ModelSpec", "Norm", "PageSpec", "PageTensor", "Part", "PartSpec", "PositionEncoding", "StateSpec",
    "StepContext", "TensorSpec", "build_block", "build_model", "build_part", "register_part",
]  # fmt: skip
