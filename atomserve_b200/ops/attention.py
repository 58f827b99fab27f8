"""Paged grouped-query attention over cache pages for a flat batch of requests."""

from __future__ import annotations

import ctypes
import functools
import os

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream

KEY_TILE = 32
TARGET_BLOCKS = 296  # two blocks for each of the 148 SMs before the key range is split
SHORT_ROWS = 8  # requests with at most this many new tokens run row by row in the decode kernel
MIXED_SCRATCH_BYTES = 128 << 20  # most that a mixed step's partial results may take (see _paged_attention_mma)


# Which kernel serves prompt portions in bfloat16 with head size 128: "tcgen05" (scores and output
# in tensor memory; the default where its shape rules hold) or "mma" (the mma.sync kernel).
PREFILL_KERNEL = os.environ.get("ATOMSERVE_B200_PREFILL_ATTENTION", "tcgen05")


# In a step that holds prompt portions and single tokens, the two attention kernels touch disjoint
# rows and neither fills the device (a portion of a few hundred tokens is one block per SM or
# fewer; a few dozen single tokens are short chains of key tiles), so the single tokens' kernels
# run on a second stream beside the portions' kernel. "0" keeps them on one stream.
MIXED_OVERLAP = os.environ.get("ATOMSERVE_B200_MIXED_OVERLAP", "1") != "0"
_SIDE: dict[torch.device, tuple] = {}  # device -> (second stream, fork event, join event)


def _side_stream(device: torch.device):
    if device not in _SIDE:
        with torch.cuda.device(device):
            _SIDE[device] = (torch.cuda.Stream(), torch.cuda.Event(), torch.cuda.Event())
    return _SIDE[device]


def attention_tile_shape(group: int) -> tuple[int, int]:
    """(tokens per query tile, query heads per block) for `group` query heads per kv head."""
    qt, gc = ctypes.c_int(), ctypes.c_int()
    lib().asb_attention_tile_shape(group, ctypes.byref(qt), ctypes.byref(gc))
    return qt.value, gc.value


def plan_partitions(num_tokens: int, num_requests: int, num_kv_heads: int, group: int,
                    max_context: int, window: int) -> tuple[int, int]:  # fmt: skip
    """(partition size, partitions): split the keys only when the batch alone cannot fill the GPU.

    Partitions are aligned to absolute key positions, so the choice never changes which keys a
    row sees, only how its sum is grouped."""
    qt, gc = attention_tile_shape(group)
    blocks = (-(-num_tokens // qt) + num_requests) * num_kv_heads * -(-group // gc)
    span = max_context if window <= 0 else min(max_context, window + qt - 1)
    if blocks >= TARGET_BLOCKS or span <= 256:
        return 1 << 30, 1
    want = -(-TARGET_BLOCKS // blocks)
    size = max(256, -(-(-(-span // want)) // 256) * 256)
    if window <= 0:
        parts = (max_context - 1) // size + 1
    else:
        parts = min((max_context - 1) // size + 1, -(-span // size) + 1)
    return (size, parts) if parts > 1 else (1 << 30, 1)


@functools.lru_cache(maxsize=4096)
def plan_decode_partitions(rows: int, num_kv_heads: int, group: int, max_context: int, window: int,
                           head_dim: int = 128) -> tuple[int, int]:  # fmt: skip
    """(partition size, partitions) for the tensor-core decode kernel, one block per (row, kv
    head, partition). The device holds a fixed number of its blocks at once, so the blocks run in
    waves; the choice minimises waves x (64-key tiles per block + 3 tiles' worth of start-up) plus
    half a tile per partition for the merge, which is what a sweep over batch 4-128 and context
    1k-8k fitted: small batches want one nearly full wave, large ones two to five, and a count
    that spills a few blocks into one more wave is the worst. Never below one tile of 64 keys a
    block (which only short contexts at small batches choose: batch 1 at 512 keys runs 8.2 us with
    four partitions of 128 against 10.3 us with two of 256)."""
    blocks = rows * num_kv_heads * -(-group // 16)
    span = max_context if window <= 0 else min(max_context, window)
    resident = lib().asb_decode_attention_resident_blocks(head_dim) or 3 * 148
    best = None
    for want in range(1, max(1, span // 64) + 1):
        size = max(64, -(-(-(-span // want)) // 64) * 64)
        if window <= 0:
            parts = (max_context - 1) // size + 1
        else:
            parts = min((max_context - 1) // size + 1, -(-span // size) + 1)
        waves = -(-blocks * parts // resident)
        cost = waves * (size // 64 + 3) + 0.5 * parts
        if best is None or cost < best[0]:
            best = (cost, size, parts)
        if want > 64:
            break
    _, size, parts = best
    return (size, parts) if parts > 1 else (1 << 30, 1)


def paged_attention(
    q: torch.Tensor,
    k_cache: torch.Tensor,
    v_cache: torch.Tensor,
    block_tables: torch.Tensor,
    req_q_start: torch.Tensor,
    req_pos_start: torch.Tensor,
    *,
    num_requests: int,
    max_context: int,
    window: int | None,
    scale: float,
    partitions: tuple[int, int] | None = None,
    host_q_lens: list[int] | None = None,
    generic: bool = False,
) -> torch.Tensor:
    """softmax(q k^T * scale) v for every new token, keys read in place from the pages.

    q: [T, H, hd]; k_cache, v_cache: [num_blocks, KV, block_size, hd]; block_tables: [R, W]
    int32; req_q_start: [R + 1] int32 (rows of each request in q); req_pos_start: [R] int32.
    max_context: the largest position + 1 any request reaches in this step (host int).
    A query at position p sees keys j <= p of its request, and j > p - window with a window.

    bfloat16 with head size 64 or 128 runs the tensor-core kernels (decode kernel for requests
    that bring at most 8 tokens, prefill kernel for longer portions; `host_q_lens`, the tokens
    each request brings, tells which are needed); everything else, and `generic=True`, runs the
    general CUDA-core kernel.
    """
    require_cuda(q, k_cache, v_cache, block_tables, req_q_start, req_pos_start)
    T, H, hd = q.shape
    KV, bs = k_cache.shape[1], k_cache.shape[2]
    if not q.is_contiguous() or k_cache.shape != v_cache.shape or k_cache.shape[3] != hd:
        raise KernelLibraryError("paged_attention: q must be contiguous and the caches [blocks, KV, bs, hd]")
    if k_cache.dtype != q.dtype or v_cache.dtype != q.dtype:
        raise KernelLibraryError("paged_attention: cache and query dtypes differ")
    for t in (block_tables, req_q_start, req_pos_start):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelLibraryError("paged_attention: index tensors must be contiguous int32")
    win = int(window) if window else 0
    out = torch.empty_like(q)
    if q.dtype == torch.bfloat16 and not generic and lib().asb_attention_mma_supported(hd, H // KV):
        return _paged_attention_mma(q, out, k_cache, v_cache, block_tables, req_q_start, req_pos_start,
                                    num_requests, max_context, win, scale, partitions, host_q_lens)  # fmt: skip
    ps, np_ = partitions or plan_partitions(T, num_requests, KV, H // KV, max_context, win)
    part_m = part_l = part_acc = None
    if np_ > 1:
        part_m = torch.empty(T * H * np_, device=q.device, dtype=torch.float32)
        part_l = torch.empty_like(part_m)
        part_acc = torch.empty(T * H * np_ * hd, device=q.device, dtype=torch.float32)
    check(lib().asb_paged_attention(
        ptr(out), ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_tables), ptr(req_q_start),
        ptr(req_pos_start), ptr(part_m), ptr(part_l), ptr(part_acc), T, num_requests, H, KV, hd, bs,
        block_tables.shape[1], win, ps, np_, float(scale), dtype_code(q), stream()))  # fmt: skip
    return out


def _paged_attention_mma(q, out, k_cache, v_cache, block_tables, req_q_start, req_pos_start, num_requests,
                         max_context, win, scale, partitions, host_q_lens):  # fmt: skip
    T, H, hd = q.shape
    KV, bs = k_cache.shape[1], k_cache.shape[2]
    if host_q_lens is None:
        has_short = has_long = True
        all_single = False
        short_rows = T
    else:
        has_short = any(n <= SHORT_ROWS for n in host_q_lens)
        has_long = any(n > SHORT_ROWS for n in host_q_lens)
        all_single = all(n == 1 for n in host_q_lens)
        short_rows = sum(n for n in host_q_lens if n <= SHORT_ROWS)
    if has_long and PREFILL_KERNEL == "tcgen05" and lib().asb_attention_tcgen05_supported(hd, H // KV, bs):
        from atomserve_b200.ops.linear import gemm_status

        def portions():
            check(lib().asb_prefill_attention_tcgen05(
                ptr(out), ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_tables), ptr(req_q_start), ptr(req_pos_start),
                T, num_requests, H, KV, hd, bs, k_cache.shape[0], block_tables.shape[1], win, float(scale),
                ptr(gemm_status(q.device)), stream()))  # fmt: skip

        if not has_short:
            portions()
            return out
        # What is left for the decode kernel: the short rows, with the key partitions their number
        # and context call for (a decoding request beside a prompt portion has as long a context
        # as in a step of its own). When the caller says how many tokens each request brings, the
        # kernel starts blocks for the short rows only and the partial results hold only those
        # rows; otherwise blocks start for every row of the step and the portions' leave at once.
        ps, np_ = partitions or plan_decode_partitions(short_rows, KV, H // KV, max_context, win, hd)
        compact = short_rows if host_q_lens is not None else 0
        scratch_rows = compact or T
        if partitions is None and scratch_rows * H * np_ * (hd + 2) * 4 > MIXED_SCRATCH_BYTES:
            ps, np_ = 1 << 30, 1
        part_m = part_l = part_acc = None
        if np_ > 1:
            part_m = torch.empty(scratch_rows * H * np_, device=q.device, dtype=torch.float32)
            # (without the short rows' count the merge runs over every row of the step and leaves
            # alone those whose sums are zero: the portions' rows, stored by their own kernel)
            part_l = (torch.empty if compact else torch.zeros)(scratch_rows * H * np_, device=q.device, dtype=torch.float32)
            part_acc = torch.empty(scratch_rows * H * np_ * hd, device=q.device, dtype=torch.float32)

        def single_tokens():
            check(lib().asb_paged_attention_mma(
                ptr(out), ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_tables), ptr(req_q_start),
                ptr(req_pos_start), ptr(part_m), ptr(part_l), ptr(part_acc), T, num_requests, H, KV, hd, bs,
                block_tables.shape[1], win, ps, np_, float(scale), 1, 0, 0, compact, stream()))  # fmt: skip
            if np_ > 1 and compact:
                check(lib().asb_attention_reduce_short(ptr(out), ptr(part_m), ptr(part_l), ptr(part_acc), ptr(req_q_start),
                                                       num_requests, SHORT_ROWS, compact, H, np_, hd, dtype_code(q), stream()))  # fmt: skip
            elif np_ > 1:
                check(lib().asb_attention_reduce(ptr(out), ptr(part_m), ptr(part_l), ptr(part_acc), T * H, np_, hd,
                                                 dtype_code(q), stream()))  # fmt: skip

        if not MIXED_OVERLAP or torch.cuda.is_current_stream_capturing():
            portions()
            single_tokens()
            return out
        # Fork: the second stream starts from what this stream has done so far (q, the cache pages,
        # the scratch), runs the single tokens, and this stream goes on only when both are done.
        # The scratch is this stream's memory; it is given back after the join, so nothing that
        # reuses it can run before the second stream has finished with it.
        main = torch.cuda.current_stream(q.device)
        side, fork, join = _side_stream(q.device)
        fork.record(main)
        portions()
        with torch.cuda.stream(side):
            side.wait_event(fork)
            single_tokens()
            join.record(side)
        main.wait_event(join)
        return out
    ps, np_ = 1 << 30, 1
    if has_short and not has_long:
        ps, np_ = partitions or plan_decode_partitions(short_rows, KV, H // KV, max_context, win, hd)
    part_m = part_l = part_acc = None
    if np_ > 1:
        part_m = torch.empty(T * H * np_, device=q.device, dtype=torch.float32)
        part_l = torch.empty_like(part_m)
        part_acc = torch.empty(T * H * np_ * hd, device=q.device, dtype=torch.float32)
    check(lib().asb_paged_attention_mma(
        ptr(out), ptr(q), ptr(k_cache), ptr(v_cache), ptr(block_tables), ptr(req_q_start),
        ptr(req_pos_start), ptr(part_m), ptr(part_l), ptr(part_acc), T, num_requests, H, KV, hd, bs,
        block_tables.shape[1], win, ps, np_, float(scale), int(has_short), int(has_long), int(all_single), 0,
        stream()))  # fmt: skip
    if np_ > 1:
        check(lib().asb_attention_reduce(ptr(out), ptr(part_m), ptr(part_l), ptr(part_acc), T * H, np_, hd,
                                         dtype_code(q), stream()))  # fmt: skip
    return out
