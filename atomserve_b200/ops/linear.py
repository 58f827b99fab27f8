"""y = x W^T (+ residual), weights in checkpoint layout [out_features, in_features].

float32 operands run this package's CUDA-core kernel with float32 multiply-adds (no tensor-core
mode of reduced precision). bfloat16 operands run this package's tcgen05 kernel (TMA operands,
float32 accumulator in tensor memory; csrc/gemm_tcgen05.cu). The vendor GEMM library through
torch, which is what the reference engine uses for its matrix products
(atomserve/quant.py:89-91), stays selectable for comparison and takes the shapes the kernel
refuses. The float32 result form (`out_dtype=torch.float32`, for logits) stores the float32
accumulator, so logits are never rounded to bfloat16.
"""

from __future__ import annotations

import ctypes
import dataclasses
import os

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream
from atomserve_b200.ops.status import status_for


def gemm_simt(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None, out_dtype: torch.dtype,
              out: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, device=x.device, dtype=out_dtype)
    check(lib().asb_gemm_simt(ptr(out), ptr(x), ptr(w), ptr(residual), M, N, K, dtype_code(x),
                              dtype_code(out), stream()))  # fmt: skip
    return out


# Which bfloat16 GEMM serves: "tcgen05" (this package's kernel, the default) or "library" (the
# vendor GEMM through torch), for comparison. Shapes the kernel refuses (K not a multiple of 8,
# unaligned operands) go to the library either way.
BACKEND = os.environ.get("ATOMSERVE_B200_GEMM", "tcgen05")

def gemm_status(device: torch.device) -> torch.Tensor:
    """The device word a tcgen05 kernel sets if one of its pipeline waits runs out."""
    return status_for(device).pipeline


def check_gemm_status(device: torch.device | str = "cuda") -> None:
    """Raise if any kernel since the last check reported through the device's status words (a
    tcgen05 wait that ran out, a token id outside the embedding table). Reads the device."""
    problem = status_for(device).problem()
    if problem:
        raise KernelLibraryError(problem)


_WORKSPACE: dict[torch.device, torch.Tensor] = {}
_OUTGROWN: list[torch.Tensor] = []


def gemm_workspace(device: torch.device, floats: int) -> torch.Tensor:
    """One float32 buffer per device for the partial sums of tensor-core GEMM calls that cut K
    (they run on one stream, one after another, so they can share it). Grown when a call needs
    more, to at least twice the size; a buffer that was outgrown is kept, not freed, because CUDA
    graphs captured while it was current still write and read their partial sums there."""
    buf = _WORKSPACE.get(device)
    if buf is None or buf.numel() < floats:
        if buf is not None:
            _OUTGROWN.append(buf)
        size = max(floats, 1 << 24, 2 * buf.numel() if buf is not None else 0)
        if torch.cuda.is_current_stream_capturing():
            # allocated here it would belong to the graph being captured and be reused by it
            raise KernelLibraryError(
                f"the GEMM workspace must grow to {size} floats during a graph capture: run the step once outside capture first"
            )
        buf = torch.zeros(size, device=device, dtype=torch.float32)
        _WORKSPACE[device] = buf
    return buf


_WORKSPACE_FLOATS: dict[tuple[int, int, int], int] = {}


def gemm_tcgen05(x: torch.Tensor, w: torch.Tensor, residual: torch.Tensor | None, out_dtype: torch.dtype,
                 swiglu: bool = False, out: torch.Tensor | None = None) -> torch.Tensor:  # fmt: skip
    """bfloat16 x [M, K] . w [N, K]^T on tcgen05 tensor cores (TMA operands, TMEM accumulator).
    swiglu: the rows of w alternate gate and up; returns silu(gate) * up, [M, N / 2]."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N // 2 if swiglu else N, device=x.device, dtype=out_dtype)
    need = _WORKSPACE_FLOATS.get((M, N, K))
    if need is None:
        query = lib().asb_gemm_tcgen05_workspace
        query.restype = ctypes.c_longlong
        need = _WORKSPACE_FLOATS[(M, N, K)] = query(M, N, K, None)
    workspace = gemm_workspace(x.device, need) if need else None
    check(lib().asb_gemm_tcgen05(ptr(out), ptr(x), ptr(w), ptr(residual), M, N, K, 2 if swiglu else int(out_dtype == torch.float32),
                                 ptr(workspace), ptr(gemm_status(x.device)), stream()))  # fmt: skip
    return out


@dataclasses.dataclass(frozen=True)
class PartialSums:
    """x . w^T as the tensor-core GEMM left it in its workspace when it cut K: float32 partial
    sums, a few slots per tile of 128 output columns (csrc/gemm_partials.cuh). A kernel that
    consumes the product can add the slots up itself (`partial_add_rms_norm`,
    `qk_norm_rope_store`), which saves the GEMM's reduction kernel. The workspace is shared: the
    sums are gone with the next tensor-core GEMM call, so they are consumed at once."""

    workspace: torch.Tensor
    tokens: int
    columns: int
    max_slots: int
    tile_tokens: int
    k_blocks_per_tile: int
    tiles: int
    blocks: int

    def layout(self) -> tuple[int, int, int, int, int, int]:
        """The arguments that the consuming kernels' entry points take after the workspace."""
        return (self.max_slots, self.tile_tokens, self.k_blocks_per_tile, self.tiles, self.blocks)


_PLANS: dict[tuple[int, int, int], tuple[int, ...]] = {}
# ATOMSERVE_B200_PARTIAL_SUMS=0: every product is reduced by the GEMM itself (for comparison)
PARTIAL_SUMS = os.environ.get("ATOMSERVE_B200_PARTIAL_SUMS", "1") != "0"


def _plan(M: int, N: int, K: int) -> tuple[int, ...]:
    plan = _PLANS.get((M, N, K))
    if plan is None:
        out = (ctypes.c_int * 8)()
        check(lib().asb_gemm_tcgen05_plan(M, N, K, out))
        plan = _PLANS[(M, N, K)] = tuple(out)
    return plan


def linear_partial(x: torch.Tensor, w: torch.Tensor) -> PartialSums | None:
    """x . w^T left as partial sums, or None where the product does not run that way (many
    tokens, float32, another backend): the caller then takes `linear`."""
    if not PARTIAL_SUMS or BACKEND != "tcgen05" or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not x.is_cuda:
        return None
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1] or not x.is_contiguous() or not w.is_contiguous():
        return None
    if not tcgen05_supported(x, w):
        return None
    (M, K), N = x.shape, w.shape[0]
    cuts_k, swapped, max_slots, tile_tokens, k_blocks, tiles, blocks, _pair = _plan(M, N, K)
    if not (cuts_k and swapped) or tiles * 128 < N or M > tile_tokens or tile_tokens & (tile_tokens - 1):
        return None  # (the consumers read slots of 16 to 256 token columns, a power of two)
    workspace = gemm_workspace(x.device, tiles * max_slots * 128 * tile_tokens)
    check(lib().asb_gemm_tcgen05(None, ptr(x), ptr(w), None, M, N, K, 3, ptr(workspace), ptr(gemm_status(x.device)), stream()))
    return PartialSums(workspace, M, N, max_slots, tile_tokens, k_blocks, tiles, blocks)


def gemm_timeline(buffer: torch.Tensor | None) -> None:
    """Profiling aid: while `buffer` (zeroed int64 [blocks + 1, 8] on the device; 160 rows are
    enough) is set, each tensor-core GEMM call overwrites it with %globaltimer stamps in
    nanoseconds: per block entry, set-up done, dependency wait over, first stage complete, last
    MMA issued, last accumulator complete, epilogue done; and in the row after the last
    block the reduction kernel's entry, wait over and end. None switches it off."""
    fn = lib().asb_gemm_tcgen05_timeline
    fn.argtypes, fn.restype = [ctypes.c_void_p], None
    fn(ptr(buffer))


def gemm_tune(swap: int = -1, rows: int = 0, cut_last_round: bool = True) -> None:
    """Tuning aid: force how the tensor-core GEMM runs the calls that follow. swap 0: unswapped
    tiles on single SMs, 1: swapped operands, 2: tiles on pairs of SMs, -1: the planner's choice;
    rows: weight rows per unswapped tile (a multiple of 32, single SMs from 64 to 256, pairs from
    128 to 256; 0: the planner's); cut_last_round: whether the pair form may cut its last round of
    tiles along K. The plans and workspace sizes remembered per shape are forgotten, because they
    differ between the forms."""
    tune = lib().asb_gemm_tcgen05_tune
    tune.argtypes, tune.restype = [ctypes.c_int, ctypes.c_int], None
    cut = lib().asb_gemm_tcgen05_pair_tune
    cut.argtypes, cut.restype = [ctypes.c_int], None
    tune(swap, rows)
    cut(1 if cut_last_round else 0)
    _WORKSPACE_FLOATS.clear()
    _PLANS.clear()


def tcgen05_supported(x: torch.Tensor, w: torch.Tensor) -> bool:
    return x.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K] gate and up matrices as one [2I, K] matrix whose rows alternate gate_i, up_i: the
    layout `linear_swiglu` multiplies with, so that a (gate, up) pair lands in one output tile."""
    return torch.stack([gate, up], dim=1).reshape(2 * gate.shape[0], gate.shape[1]).contiguous()


def swiglu_fusable(w: torch.Tensor) -> bool:
    """Whether x . w^T with this weight can run the fused SwiGLU form of the tensor-core GEMM."""
    return BACKEND == "tcgen05" and w.dtype == torch.bfloat16 and w.shape[1] % 8 == 0 and w.data_ptr() % 16 == 0


def linear_swiglu(x: torch.Tensor, w_interleaved: torch.Tensor) -> torch.Tensor:
    """silu(x . gate^T) * (x . up^T) in one kernel: the products accumulate in float32 in tensor
    memory and the activation is applied to those sums before the one rounding to bfloat16
    (the unfused path rounds the two products first, atomserve/model.py:354-359)."""
    require_cuda(x, w_interleaved)
    if x.dtype != torch.bfloat16 or not swiglu_fusable(w_interleaved) or not x.is_contiguous() or x.data_ptr() % 16:
        raise KernelLibraryError("linear_swiglu takes contiguous bfloat16 operands with K a multiple of 8")
    return gemm_tcgen05(x, w_interleaved, None, torch.bfloat16, swiglu=True)


def linear(
    x: torch.Tensor,
    w: torch.Tensor,
    residual: torch.Tensor | None = None,
    out_dtype: torch.dtype | None = None,
    out: torch.Tensor | None = None,
) -> torch.Tensor:
    """`out`, if given, is the contiguous [M, N] tensor of the output dtype that takes the result."""
    require_cuda(x, w, residual, out)
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelLibraryError(f"linear: x {tuple(x.shape)} does not match w {tuple(w.shape)}")
    if x.dtype != w.dtype or not x.is_contiguous() or not w.is_contiguous():
        raise KernelLibraryError("linear: x and w must be contiguous and of one dtype")
    out_dtype = out_dtype or x.dtype
    if residual is not None and (residual.shape != (x.shape[0], w.shape[0]) or residual.dtype != out_dtype or not residual.is_contiguous()):
        raise KernelLibraryError("linear: residual must be [M, N], contiguous, in the output dtype")
    if out is not None and (out.shape != (x.shape[0], w.shape[0]) or out.dtype != out_dtype or not out.is_contiguous()):
        raise KernelLibraryError("linear: out must be [M, N], contiguous, in the output dtype")
    if x.dtype == torch.float32:
        if out_dtype != torch.float32:
            raise KernelLibraryError("linear: float32 operands give float32 results")
        return gemm_simt(x, w, residual, torch.float32, out)
    if out_dtype == torch.float32 and residual is not None:
        return gemm_simt(x, w, residual, torch.float32, out)
    if BACKEND == "tcgen05" and tcgen05_supported(x, w):
        return gemm_tcgen05(x, w, residual, out_dtype, out=out)
    if out_dtype == torch.float32:
        result = torch.mm(x, w.t(), out_dtype=torch.float32)  # float32 accumulator, not rounded
    elif residual is None:
        result = torch.mm(x, w.t())
    else:
        result = torch.addmm(residual, x, w.t())
    return result if out is None else out.copy_(result)
