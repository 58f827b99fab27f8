"""Loads the CUDA library and declares its C entry points.

The kernels are the only implementation of the hot operations: there is no CPU or PyTorch
stand-in behind them. If the library cannot be built or loaded, or the device is not the one
it was compiled for, the first operation raises `KernelLibraryError`.
"""

from __future__ import annotations

import ctypes
import os
import threading
from ctypes import c_float, c_int, c_void_p

import torch

_LOCK = threading.Lock()
_LIB: ctypes.CDLL | None = None

FLOAT32, BFLOAT16 = 0, 1
DTYPE_CODES = {torch.float32: FLOAT32, torch.bfloat16: BFLOAT16}


class KernelLibraryError(RuntimeError):
    """The CUDA extension is missing, unbuildable, or was refused by a kernel's size checks."""


_P, _I, _F = c_void_p, c_int, c_float
_SIGNATURES = {
    "asb_embedding": [_P, _P, _P, _I, _I, _I, _I, _P, _P],
    "asb_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _P],
    "asb_silu_mul": [_P, _P, _I, _I, _I, _P],
    "asb_qk_norm_rope_store": [_P] * 9 + [_I] * 6 + [_F, _I, _P],
    "asb_paged_attention": [_P] * 10 + [_I] * 10 + [_F, _I, _P],
    "asb_paged_attention_mma": [_P] * 10 + [_I] * 10 + [_F, _I, _I, _I, _I, _P],
    "asb_prefill_attention_tcgen05": [_P] * 7 + [_I] * 9 + [_F, _P, _P],
    "asb_attention_tcgen05_supported": [_I, _I, _I],
    "asb_attention_reduce": [_P, _P, _P, _P, _I, _I, _I, _I, _P],
    "asb_attention_reduce_short": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
    "asb_attention_mma_supported": [_I, _I],
    "asb_decode_attention_resident_blocks": [_I],
    "asb_gemm_tcgen05": [_P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P],
    "asb_gemm_tcgen05_plan": [_I, _I, _I, _P],
    "asb_partial_add_rmsnorm": [_P, _P, _P, _I, _I, _I, _I, _I, _P, _P, _I, _I, _F, _P],
    "asb_qk_norm_rope_store_partial": [_P] * 4 + [_I] * 5 + [_P] * 5 + [_I] * 6 + [_F, _P],
    "asb_gemm_simt": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _P],
    "asb_argmax_rows": [_P, _P, _I, _I, _P],
    "asb_presence_penalty": [_P, _P, _P, _P, _I, _I, _P],
    "asb_sample_rows": [_P, _P, _I, _I, _P, _P, _P, _P, _P, _P],
}


def lib() -> ctypes.CDLL:
    """The loaded library; builds it first if the tree holds no current one."""
    global _LIB
    if _LIB is not None:
        return _LIB
    with _LOCK:
        if _LIB is not None:
            return _LIB
        from atomserve_b200.csrc import build

        try:
            path = build.build()
            handle = ctypes.CDLL(str(path))
        except Exception as error:  # noqa: BLE001
            raise KernelLibraryError(
                f"the CUDA kernel library could not be built or loaded: {error}"
            ) from error
        handle.asb_last_error.restype = ctypes.c_char_p
        handle.asb_launch_count.restype = ctypes.c_longlong
        handle.asb_set_pdl.argtypes = [c_int]
        handle.asb_set_pdl.restype = None
        # programmatic dependent launch: kernels are scheduled while their predecessor drains
        handle.asb_set_pdl(int(os.environ.get("ATOMSERVE_B200_PDL", "1") != "0"))
        handle.asb_attention_tile_shape.argtypes = [c_int, c_void_p, c_void_p]
        handle.asb_attention_tile_shape.restype = None
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(handle, name, None)
            if fn is None:
                raise KernelLibraryError(f"{path} lacks the entry point {name}")
            fn.argtypes = argtypes
            fn.restype = c_int
        _LIB = handle
    return _LIB


def declare(name: str, argtypes: list) -> None:
    """Declare a further entry point (used by ops that live in their own source files)."""
    _SIGNATURES[name] = argtypes
    if _LIB is not None:
        fn = getattr(_LIB, name)
        fn.argtypes, fn.restype = argtypes, c_int


_REPLAYED = [0]  # kernels run by CUDA-graph replays: counted from what each capture recorded


def launches() -> int:
    """Kernels of this library launched so far in this process, graph replays included."""
    return int(lib().asb_launch_count()) + _REPLAYED[0]


def note_replay(kernels: int) -> None:
    _REPLAYED[0] += kernels


def check(code: int) -> None:
    if code != 0:
        raise KernelLibraryError(lib().asb_last_error().decode())


def require_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelLibraryError(
                "this operation runs only as a CUDA kernel on sm_100a; it was given a "
                f"{t.device.type} tensor (there is no CPU path)"
            )


def require_device() -> None:
    """Fail loudly when there is no CUDA device or it is not the compiled architecture."""
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: the engine has no CPU path")
    major, minor = torch.cuda.get_device_capability()
    if major != 10:
        raise KernelLibraryError(
            f"the kernels are compiled for sm_100a only; this device is sm_{major}{minor}"
        )


def dtype_code(t: torch.Tensor) -> int:
    try:
        return DTYPE_CODES[t.dtype]
    except KeyError:
        raise KernelLibraryError(f"kernels take float32 or bfloat16, not {t.dtype}") from None


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def stream() -> int:
    """The current CUDA stream's handle (called once per kernel launch, so by the cheapest route
    torch offers)."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream
