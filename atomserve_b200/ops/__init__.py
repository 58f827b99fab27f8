"""Python faces of the CUDA kernels. Each function checks its tensors, allocates the output
and launches on the current stream. float32 tensors run the true 32-bit kernels, bfloat16
tensors the serving kernels; nothing here computes on the CPU."""

from atomserve_b200.ops.attention import attention_tile_shape, paged_attention
from atomserve_b200.ops.elementwise import (
    embedding,
    partial_add_rms_norm,
    partial_add_rms_norm_fusable,
    qk_norm_rope_store,
    qk_norm_rope_store_takes_partial,
    rms_norm,
    rotary,
    silu_mul,
)
from atomserve_b200.ops.library import KernelLibraryError, require_device
from atomserve_b200.ops.linear import PartialSums, interleave_gate_up, linear, linear_partial, linear_swiglu, swiglu_fusable
from atomserve_b200.ops.sampling import argmax_rows, presence_penalty, sample_rows
from atomserve_b200.ops.status import DeviceStatus, status_for

__all__ = [
    "DeviceStatus",
    "KernelLibraryError",
    "PartialSums",
    "argmax_rows",
    "attention_tile_shape",
    "embedding",
    "interleave_gate_up",
    "linear",
    "linear_partial",
    "linear_swiglu",
    "paged_attention",
    "partial_add_rms_norm",
    "partial_add_rms_norm_fusable",
    "presence_penalty",
    "qk_norm_rope_store",
    "qk_norm_rope_store_takes_partial",
    "require_device",
    "rms_norm",
    "rotary",
    "sample_rows",
    "silu_mul",
    "status_for",
    "swiglu_fusable",
]
