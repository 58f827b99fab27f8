"""Host arithmetic that the kernels' launches rest on, checked without a GPU: the decode
attention's key partitions and the tensor-core GEMM's schedule of tiles, K ranges and partial-sum
slots."""

import pytest


def test_decode_attention_partition_plans_cover_every_context(monkeypatch):
    """The planner of the decode attention's key partitions is host arithmetic: whatever the
    batch, context and window, its partitions are whole 64-key tiles, start at multiples of their
    size and reach the last key."""
    import random

    import atomserve_b200.ops.attention as attention

    class FakeLibrary:
        def asb_decode_attention_resident_blocks(self, head_dim):
            return 444

    monkeypatch.setattr(attention, "lib", lambda: FakeLibrary())
    attention.plan_decode_partitions.cache_clear()
    rng = random.Random(0)
    for _ in range(2000):
        rows = rng.choice([1, 2, 3, 8, 17, 64, 200])
        kv, group = rng.choice([(1, 1), (2, 4), (8, 4), (4, 20)])
        context = rng.choice([1, 63, 64, 65, 300, 2048, 2088, 8191, 40000])
        window = rng.choice([0, 0, 100, 4096])
        size, parts = attention.plan_decode_partitions(rows, kv, group, context, window)
        assert parts >= 1
        if parts == 1:
            assert size >= context
            continue
        assert size % 64 == 0 and size >= 64
        if window <= 0:
            assert (parts - 1) * size < context <= parts * size
        else:
            # a row's window of keys spans at most this many partitions of that size
            assert parts <= -(-min(context, window) // size) + 1
    attention.plan_decode_partitions.cache_clear()


def test_gemm_plans_keep_every_tile_within_its_partial_sum_slots():
    """The tensor-core GEMM's schedule is host arithmetic inside the library (it needs no GPU):
    whatever the shape, the tiles cover the product, only swapped operands cut K, every block has
    at least one K block, and no tile is shared by more blocks than it has workspace slots."""
    import ctypes
    import random

    try:
        from atomserve_b200.ops.library import lib

        plan = lib().asb_gemm_tcgen05_plan
    except Exception as error:  # no compiler here, or the library does not load without a driver
        pytest.skip(f"the kernel library is not available: {error}")
    plan.argtypes = [ctypes.c_int] * 3 + [ctypes.POINTER(ctypes.c_int)]
    plan.restype = None
    pair_cut, workspace = lib().asb_gemm_tcgen05_pair_cut, lib().asb_gemm_tcgen05_workspace
    pair_cut.argtypes, pair_cut.restype = [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_int)], ctypes.c_longlong
    workspace.argtypes, workspace.restype = [ctypes.c_int] * 3 + [ctypes.POINTER(ctypes.c_int)], ctypes.c_longlong
    out, cut = (ctypes.c_int * 8)(), (ctypes.c_int * 3)()
    cut_plans = 0
    rng = random.Random(1)
    shapes = [(8, 4096, 4096), (1, 151936, 4096), (512, 4096, 12288), (2048, 24576, 4096), (300, 5120, 17408)]
    for _ in range(3000):
        shapes.append((rng.choice([1, 2, 7, 16, 17, 33, 64, 100, 129, 256, 257, 400, 512, 513, 1000, 2048, 5000]),
                       rng.choice([8, 100, 128, 130, 1000, 1024, 4096, 5120, 6144, 24576, 40000]),
                       rng.choice([8, 64, 72, 128, 1000, 4096, 8192, 12288, 17408])))  # fmt: skip
    for M, N, K in shapes:
        plan(M, N, K, out)
        cuts_k, swap, max_slots, bn, kb, tiles, blocks, pair = list(out)
        assert kb == -(-K // 64) and 1 <= blocks <= 148, (M, N, K)
        if pair:  # tiles of 256 tokens by `pair` weight rows, two blocks (a pair of SMs) on each
            assert pair in (128, 160, 192, 224, 256) and bn == pair and not swap and not cuts_k and M > 128, (M, N, K)
            assert tiles == -(-M // 256) * -(-N // pair), (M, N, K)
            # the last round of tiles may be cut along K: whole rounds first, then `split` pairs on
            # each tile left, every piece with stages to run, one workspace slot a piece
            floats = pair_cut(M, N, K, pair, cut)
            whole, split, piece = list(cut)
            stages = -(-kb // 2)
            slot = 256 * (128 if pair == 128 else 256)  # a slot is as wide as the widest tile of the kernel that runs it
            assert workspace(M, N, K, None) == floats == ((tiles - whole) * split * slot if split > 1 else 0), (M, N, K)
            if split == 1:
                assert whole == tiles and blocks == 2 * min(tiles, 74), (M, N, K)
            else:
                cut_plans += 1
                assert whole % 74 == 0 and 0 < tiles - whole and (tiles - whole) * split <= 74, (M, N, K)
                assert (split - 1) * piece < stages <= split * piece and piece >= 4, (M, N, K)
                assert blocks == 2 * (74 if whole else tiles * split), (M, N, K)
            continue
        p_rows, q_rows = (N, M) if swap else (M, N)
        assert tiles == -(-p_rows // 128) * -(-q_rows // bn), (M, N, K)
        assert bn in (16, 32, 64, 128, 256) if swap else (bn % 32 == 0 and 64 <= bn <= 256), (M, N, K, bn)
        if swap:
            assert bn >= min(M, 256) or M > 256, (M, N, K, bn)
        if not cuts_k:
            assert blocks == min(tiles, 148), (M, N, K)
            continue
        assert swap, (M, N, K)
        total = tiles * kb
        begins = [total * c // blocks for c in range(blocks + 1)]
        assert all(b1 > b0 for b0, b1 in zip(begins, begins[1:])), (M, N, K)  # no empty range
        import bisect

        for tile in range(tiles):
            first = bisect.bisect_right(begins, tile * kb) - 1
            last = bisect.bisect_right(begins, tile * kb + kb - 1) - 1
            assert last - first + 1 <= max_slots, (M, N, K, tile)
    assert cut_plans > 20


def test_decode_graph_keys_are_few_and_the_cache_of_graphs_is_bounded():
    """Decode graphs are keyed by (batch bucket, table-width bucket, context bucket): over every
    batch up to 256 and every context up to 40k the buckets stay few, each rounds up by little,
    and the cache that holds the captured graphs never grows beyond its limit."""
    from atomserve_b200.engine.runner import GraphCache, batch_bucket, context_bucket, width_bucket

    assert batch_bucket(257) is None
    batches = {batch_bucket(b) for b in range(1, 257)}
    assert len(batches) <= 16 and all(batch_bucket(b) >= b for b in range(1, 257))
    contexts = set()
    for ctx in range(1, 40961, 7):
        bucket = context_bucket(ctx)
        assert ctx <= bucket and (bucket - ctx < 256 or bucket <= ctx * 1.25)
        contexts.add(bucket)
    assert len(contexts) <= 64
    assert {width_bucket(p) for p in range(1, 2561)} == {16, 32, 64, 128, 256, 512, 1024, 2048, 4096}
    cache = GraphCache(limit=48)
    dropped = 0
    for b in sorted(batches):
        for ctx in sorted(contexts):
            key = (b, b, (width_bucket(-(-ctx // 16)),), b, ctx)
            if cache.get(key) is None:
                cache.put(key, ("graph", 0))
            assert len(cache) <= 48
    assert cache.get((1, 1, (16,), 1, 256)) is None  # the oldest went first
    recent = (256, 256, (width_bucket(40960 // 16),), 256, 40960)
    assert cache.get(recent) is not None
    cache.put(("x",), ("graph", 0))
    assert cache.get(recent) is not None and len(cache) == 48
