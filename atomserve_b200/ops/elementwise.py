"""Embedding, RMSNorm, the fused q/k-norm + rotary + cache write, and SiLU*up."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream
from atomserve_b200.ops.linear import PartialSums


def _int32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.int32 or not t.is_contiguous():
        raise KernelLibraryError(f"{name} must be a contiguous int32 tensor, got {t.dtype}")


def _gain(t: torch.Tensor | None, n: int, name: str) -> None:
    if t is not None and (t.dtype != torch.float32 or t.shape != (n,) or not t.is_contiguous()):
        raise KernelLibraryError(f"{name} must be float32 of shape [{n}], got {t.dtype} {tuple(t.shape)}")


def embedding(ids: torch.Tensor, table: torch.Tensor, status: torch.Tensor) -> torch.Tensor:
    """out[t] = table[ids[t]]. ids: [T] int32; table: [V, d]; status: int32[1], set to 1 by an
    id outside the table (the row is then zero)."""
    require_cuda(ids, table, status)
    _int32(ids, "ids")
    _int32(status, "status")
    if table.dim() != 2 or not table.is_contiguous():
        raise KernelLibraryError("embedding table must be a contiguous matrix")
    out = torch.empty(ids.shape[0], table.shape[1], device=table.device, dtype=table.dtype)
    check(lib().asb_embedding(ptr(out), ptr(table), ptr(ids), ids.shape[0], table.shape[1],
                              table.shape[0], dtype_code(table), ptr(status), stream()))  # fmt: skip
    return out


def rms_norm(x: torch.Tensor, gain: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> torch.Tensor:
    """gain * x / sqrt(mean(x^2) + eps) over the last dim of x [N, d]; with `rows` (int32 [n])
    only those rows of x are normalised and returned, in that order."""
    require_cuda(x, gain, rows)
    if x.dim() != 2 or not x.is_contiguous():
        raise KernelLibraryError("rms_norm takes a contiguous [rows, width] tensor")
    _gain(gain, x.shape[1], "gain")
    n = x.shape[0]
    if rows is not None:
        _int32(rows, "rows")
        n = rows.shape[0]
    out = torch.empty(n, x.shape[1], device=x.device, dtype=x.dtype)
    check(lib().asb_rmsnorm(ptr(out), ptr(x), ptr(gain), ptr(rows), n, x.shape[1], float(eps),
                            dtype_code(x), stream()))  # fmt: skip
    return out


def partial_add_rms_norm_fusable(width: int) -> bool:
    return width % 8 == 0 and width <= 8192


def partial_add_rms_norm(product: PartialSums, residual: torch.Tensor | None, gain: torch.Tensor,
                         eps: float) -> tuple[torch.Tensor, torch.Tensor]:  # fmt: skip
    """(product + residual, rms_norm(product + residual)) in one kernel, the product given as the
    GEMM's partial sums. The same bits as `linear(..., residual)` followed by `rms_norm`."""
    require_cuda(residual, gain)
    T, N = product.tokens, product.columns
    if not partial_add_rms_norm_fusable(N):
        raise KernelLibraryError(f"partial_add_rms_norm: width {N} is not taken (a multiple of 8 up to 8192)")
    _gain(gain, N, "gain")
    if residual is not None and (residual.shape != (T, N) or residual.dtype != torch.bfloat16 or not residual.is_contiguous()):
        raise KernelLibraryError("partial_add_rms_norm: residual must be a contiguous bfloat16 [tokens, width] tensor")
    total = torch.empty(T, N, device=gain.device, dtype=torch.bfloat16)
    normed = torch.empty_like(total)
    check(lib().asb_partial_add_rmsnorm(ptr(total), ptr(normed), ptr(product.workspace), *product.layout(),
                                        ptr(residual), ptr(gain), T, N, float(eps), stream()))  # fmt: skip
    return total, normed


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """[T, 2I] (gate columns first, then up) -> silu(gate) * up, [T, I]."""
    require_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelLibraryError("silu_mul takes a contiguous [tokens, 2 * intermediate] tensor")
    inter = gate_up.shape[1] // 2
    out = torch.empty(gate_up.shape[0], inter, device=gate_up.device, dtype=gate_up.dtype)
    check(lib().asb_silu_mul(ptr(out), ptr(gate_up), gate_up.shape[0], inter, dtype_code(gate_up), stream()))
    return out


def qk_norm_rope_store_takes_partial(head_dim: int, rotary_dim: int | None) -> bool:
    """Whether `qk_norm_rope_store` can read its qkv from the GEMM's partial sums."""
    return head_dim in (32, 64, 128, 256) and rotary_dim in (None, 0, head_dim)


def qk_norm_rope_store(
    qkv: torch.Tensor | PartialSums,
    num_heads: int,
    num_kv_heads: int,
    head_dim: int,
    positions: torch.Tensor,
    *,
    q_gain: torch.Tensor | None,
    k_gain: torch.Tensor | None,
    eps: float,
    inv_freq: torch.Tensor | None,
    rotary_dim: int,
    slots: torch.Tensor | None,
    k_cache: torch.Tensor | None,
    v_cache: torch.Tensor | None,
) -> torch.Tensor:
    """Normalise and rotate q and k heads and store k, v into cache pages; returns q [T, H, hd].

    qkv: [T, (H + 2 KV) * hd], heads ordered q | k | v. k_cache, v_cache: one cache entry,
    [num_blocks, KV, block_size, hd]; slots: [T] int32 (block * block_size + offset, negative:
    not stored). With num_kv_heads == 0 only q heads are present and nothing is stored.
    """
    partial = qkv if isinstance(qkv, PartialSums) else None
    if partial is not None:
        require_cuda(positions, q_gain, k_gain, inv_freq, slots, k_cache, v_cache)
        T, width, dtype, device = partial.tokens, partial.columns, torch.bfloat16, partial.workspace.device
        if not qk_norm_rope_store_takes_partial(head_dim, rotary_dim if inv_freq is not None else None):
            raise KernelLibraryError(f"qk_norm_rope_store: head_dim {head_dim} with rotary_dim {rotary_dim} is not read from partial sums")
    else:
        require_cuda(qkv, positions, q_gain, k_gain, inv_freq, slots, k_cache, v_cache)
        T, width, dtype, device = qkv.shape[0], qkv.shape[1] if qkv.dim() == 2 else -1, qkv.dtype, qkv.device
        if not qkv.is_contiguous():
            width = -1
    if width != (num_heads + 2 * num_kv_heads) * head_dim:
        raise KernelLibraryError(f"qkv has width {width}, expected [T, {(num_heads + 2 * num_kv_heads) * head_dim}] contiguous")
    _int32(positions, "positions")
    _gain(q_gain, head_dim, "q_gain")
    _gain(k_gain, head_dim, "k_gain")
    if inv_freq is not None:
        _gain(inv_freq, rotary_dim // 2, "inv_freq")
    block_size = 1
    if num_kv_heads > 0 and slots is not None:
        _int32(slots, "slots")
        for c in (k_cache, v_cache):
            if c is None or c.dtype != dtype or c.dim() != 4 or c.shape[1] != num_kv_heads or c.shape[3] != head_dim or not c.is_contiguous():
                raise KernelLibraryError("cache entry must be [num_blocks, KV, block_size, head_dim] in the activations' dtype")
        block_size = k_cache.shape[2]
    q = torch.empty(T, num_heads, head_dim, device=device, dtype=dtype)
    if partial is not None:
        check(lib().asb_qk_norm_rope_store_partial(
            ptr(q), ptr(k_cache), ptr(v_cache), ptr(partial.workspace), *partial.layout(), ptr(q_gain), ptr(k_gain),
            ptr(inv_freq), ptr(positions), ptr(slots), T, num_heads, num_kv_heads, head_dim, rotary_dim, block_size,
            float(eps), stream()))  # fmt: skip
        return q
    check(lib().asb_qk_norm_rope_store(
        ptr(q), ptr(k_cache), ptr(v_cache), ptr(qkv), ptr(q_gain), ptr(k_gain), ptr(inv_freq),
        ptr(positions), ptr(slots), T, num_heads, num_kv_heads, head_dim, rotary_dim, block_size,
        float(eps), dtype_code(qkv), stream()))  # fmt: skip
    return q


def rotary(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, rotary_dim: int) -> torch.Tensor:
    """Rotate-half rotary encoding of x [T, heads, hd] alone (no norm, no store)."""
    T, heads, hd = x.shape
    return qk_norm_rope_store(
        x.reshape(T, heads * hd), heads, 0, hd, positions, q_gain=None, k_gain=None, eps=0.0,
        inv_freq=inv_freq, rotary_dim=rotary_dim, slots=None, k_cache=None, v_cache=None,
    )  # fmt: skip
