"""Each CUDA kernel alone against its plain reference, at sizes other than the engine's."""

import math

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


@pytest.fixture(scope="module")
def ops():
    from atomserve_b200 import ops

    ops.require_device()
    return ops


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [48, 100, 4096])
def test_embedding(ops, dtype, width):
    table = torch.randn(331, width, device="cuda").to(dtype)
    ids = torch.tensor([0, 330, 7, 7, 19], dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = ops.embedding(ids, table, status)
    assert torch.equal(out, table[ids.long()])
    assert int(status) == 0
    bad = torch.tensor([3, 331], dtype=torch.int32, device="cuda")
    out = ops.embedding(bad, table, status)
    assert int(status) == 1 and torch.equal(out[1], torch.zeros_like(out[1]))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,width,eps", [(1, 16, 1e-6), (7, 100, 1e-5), (33, 4096, 1e-6), (3, 5120, 3e-6)])
def test_rms_norm(ops, dtype, rows, width, eps):
    x = (torch.randn(rows, width, device="cuda") * 3).to(dtype)
    gain = 1 + 0.1 * torch.randn(width, device="cuda")
    ref = plain.rms_norm(x.float().cpu(), gain.cpu(), eps)
    out = ops.rms_norm(x, gain, eps)
    assert torch.allclose(out.float().cpu(), ref, **tol(dtype))
    pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device="cuda")
    out = ops.rms_norm(x, gain, eps, pick)
    assert torch.allclose(out.float().cpu(), ref[[rows - 1, 0]], **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,inter", [(1, 24), (7, 176), (300, 12288)])
def test_silu_mul(ops, dtype, rows, inter):
    gu = (torch.randn(rows, 2 * inter, device="cuda") * 2).to(dtype)
    g, u = gu.float().cpu()[:, :inter], gu.float().cpu()[:, inter:]
    ref = g / (1 + torch.exp(-g)) * u
    assert torch.allclose(ops.silu_mul(gu).float().cpu(), ref, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 64, 64), (5, 100, 37), (70, 130, 259), (128, 512, 1024)])
def test_linear(ops, dtype, M, N, K):
    x = torch.randn(M, K, device="cuda").to(dtype)
    w = (torch.randn(N, K, device="cuda") / math.sqrt(K)).to(dtype)
    res = torch.randn(M, N, device="cuda").to(dtype)
    ref = x.double().cpu() @ w.double().cpu().T
    t = dict(atol=1e-5, rtol=1e-5) if dtype == torch.float32 else dict(atol=3e-2, rtol=2e-2)
    assert torch.allclose(ops.linear(x, w).double().cpu(), ref, **t)
    assert torch.allclose(ops.linear(x, w, res).double().cpu(), ref + res.double().cpu(), **t)
    full = ops.linear(x, w, out_dtype=torch.float32)
    assert full.dtype == torch.float32
    assert torch.allclose(full.double().cpu(), ref, atol=1e-3 if dtype == torch.bfloat16 else 1e-5, rtol=1e-3)


def test_linear_rows_do_not_depend_on_the_batch(ops):
    """float32: a row's result is bit-equal whether it runs alone or among others."""
    x = torch.randn(70, 259, device="cuda")
    w = torch.randn(130, 259, device="cuda")
    whole = ops.linear(x, w)
    assert torch.equal(ops.linear(x[17:18].contiguous(), w), whole[17:18])
    assert torch.equal(ops.linear(x[60:].contiguous(), w), whole[60:])


def rope_reference(x, positions, hd, theta, rotary_dim=None):
    rd = rotary_dim or hd
    angles = plain.rope_angles(positions, rd, theta)
    rotated = plain.apply_rope(x[..., :rd], angles)
    return torch.cat([rotated, x[..., rd:]], dim=-1)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,rd,theta", [(16, 16, 1e4), (48, 48, 5e4), (128, 128, 1e6), (256, 64, 1e4), (32, 32, 1e4),
                                         (64, 64, 1e6), (256, 256, 5e5)])  # fmt: skip
def test_rotary_alone(ops, dtype, hd, rd, theta):
    from atomserve_b200.parts.rotary import Rotary

    rot = Rotary(hidden_size=0, prefix="", head_dim=hd, theta=theta, rotary_dim=rd)
    rot.prepare(torch.device("cuda"))
    pos = torch.tensor([0, 1, 300, 4097, 39999], dtype=torch.int32, device="cuda")
    x = torch.randn(5, 3, hd, device="cuda").to(dtype)
    ref = rope_reference(x.float().cpu(), pos.cpu().long(), hd, theta, rd)
    out = rot.apply(x, pos)
    assert torch.allclose(out.float().cpu(), ref, **(dict(atol=2e-4, rtol=1e-4) if dtype == torch.float32 else tol(dtype)))
    assert torch.equal(out[0], x[0])  # position 0 is the identity


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd,bs", [(4, 2, 16, 16), (5, 1, 48, 8), (32, 8, 128, 16), (16, 16, 80, 4), (6, 3, 32, 8),
                                        (9, 3, 64, 16), (4, 4, 256, 8)])  # fmt: skip
def test_qk_norm_rope_store(ops, dtype, H, KV, hd, bs):
    T, nblocks, eps, theta = 6, 9, 1e-5, 1e6
    qkv = torch.randn(T, (H + 2 * KV) * hd, device="cuda").to(dtype)
    qg, kg = (1 + 0.1 * torch.randn(hd, device="cuda") for _ in range(2))
    inv_freq = plain.rope_inv_freq(hd, theta).cuda()
    pos = torch.tensor([0, 1, 300, 4097, 39999, 17], dtype=torch.int32, device="cuda")
    slot_list = [bs * 7 + 1, 0, bs * 3 + bs - 1, 5 % bs + bs * 2, bs * 8, -1]
    slots = torch.tensor(slot_list, dtype=torch.int32, device="cuda")
    kc = torch.zeros(nblocks, KV, bs, hd, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    q = ops.qk_norm_rope_store(qkv, H, KV, hd, pos, q_gain=qg, k_gain=kg, eps=eps, inv_freq=inv_freq,
                               rotary_dim=hd, slots=slots, k_cache=kc, v_cache=vc)  # fmt: skip
    x = qkv.float().cpu().view(T, H + 2 * KV, hd)
    angles = plain.rope_angles(pos.cpu().long(), hd, theta)
    q_ref = plain.apply_rope(plain.rms_norm(x[:, :H], qg.cpu(), eps), angles)
    k_ref = plain.apply_rope(plain.rms_norm(x[:, H : H + KV], kg.cpu(), eps), angles)
    t = dict(atol=3e-4, rtol=1e-4) if dtype == torch.float32 else tol(dtype)
    assert torch.allclose(q.float().cpu(), q_ref, **t)
    kflat = kc.float().cpu().permute(0, 2, 1, 3).reshape(nblocks * bs, KV, hd)
    vflat = vc.cpu().permute(0, 2, 1, 3).reshape(nblocks * bs, KV, hd)
    written = [s for s in slot_list if s >= 0]
    for i, s in enumerate(slot_list):
        if s >= 0:
            assert torch.allclose(kflat[s], k_ref[i], **t)
            assert torch.equal(vflat[s], qkv.cpu().view(T, H + 2 * KV, hd)[i, H + KV :])  # v bit-equal
    untouched = torch.ones(nblocks * bs, dtype=torch.bool)
    untouched[written] = False
    assert float(kflat[untouched].abs().max()) == 0 and float(vflat[untouched].float().abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,KV,hd,bs,gains", [(32, 8, 128, 16, True), (5, 1, 64, 8, True), (3, 3, 256, 4, False),
                                              (6, 2, 32, 16, True), (7, 1, 48, 8, True)])  # fmt: skip
def test_qk_norm_rope_store_many_tokens(ops, dtype, H, KV, hd, bs, gains):
    """The forms that portions of hundreds of tokens take (a block per token, several heads a
    warp), at head counts that leave warps half used, with some tokens not stored."""
    T, eps, theta = 300, 1e-6, 5e5
    g = torch.Generator().manual_seed(hd + H)
    qkv = torch.randn(T, (H + 2 * KV) * hd, generator=g).cuda().to(dtype)
    qg, kg = ((1 + 0.1 * torch.randn(hd, generator=g)).cuda() if gains else None for _ in range(2))
    inv_freq = plain.rope_inv_freq(hd, theta).cuda()
    pos = torch.randint(0, 30000, (T,), generator=g).int().cuda()
    nblocks = T // bs + 3
    slot_list = torch.randperm(nblocks * bs, generator=g)[:T].tolist()
    for i in range(0, T, 7):
        slot_list[i] = -1
    slots = torch.tensor(slot_list, dtype=torch.int32, device="cuda")
    kc = torch.zeros(nblocks, KV, bs, hd, device="cuda", dtype=dtype)
    vc = torch.zeros_like(kc)
    q = ops.qk_norm_rope_store(qkv, H, KV, hd, pos, q_gain=qg, k_gain=kg, eps=eps if gains else 0.0, inv_freq=inv_freq,
                               rotary_dim=hd, slots=slots, k_cache=kc, v_cache=vc)  # fmt: skip
    x = qkv.float().cpu().view(T, H + 2 * KV, hd)
    angles = plain.rope_angles(pos.cpu().long(), hd, theta)
    normed = (lambda v, gain: plain.rms_norm(v, gain.cpu(), eps)) if gains else (lambda v, gain: v)
    q_ref = plain.apply_rope(normed(x[:, :H], qg), angles)
    k_ref = plain.apply_rope(normed(x[:, H : H + KV], kg), angles)
    t = dict(atol=3e-4, rtol=1e-4) if dtype == torch.float32 else tol(dtype)
    assert torch.allclose(q.float().cpu(), q_ref, **t)
    kflat = kc.float().cpu().permute(0, 2, 1, 3).reshape(nblocks * bs, KV, hd)
    vflat = vc.cpu().permute(0, 2, 1, 3).reshape(nblocks * bs, KV, hd)
    stored = torch.tensor([s >= 0 for s in slot_list])
    at = torch.tensor([s for s in slot_list if s >= 0])
    assert torch.allclose(kflat[at], k_ref[stored], **t)
    assert torch.equal(vflat[at], qkv.cpu().view(T, H + 2 * KV, hd)[stored][:, H + KV :])
    untouched = torch.ones(nblocks * bs, dtype=torch.bool)
    untouched[at] = False
    assert float(kflat[untouched].abs().max()) == 0 and float(vflat[untouched].float().abs().max()) == 0


def paged_setup(ctx_lens, q_lens, H, KV, hd, bs, dtype, seed=0, special=None):
    """Random q/k/v for R requests; keys/values scattered over shuffled pages. Returns device
    inputs and the dense per-request k, v for the reference. `special` = (request, position):
    that key and the request's last query are made to match strongly."""
    g = torch.Generator().manual_seed(seed)
    R = len(ctx_lens)
    nblocks = sum(-(-c // bs) for c in ctx_lens) + 3
    order = torch.randperm(nblocks, generator=g).tolist()
    kc = torch.zeros(nblocks, KV, bs, hd)
    vc = torch.zeros(nblocks, KV, bs, hd)
    width = max(-(-c // bs) for c in ctx_lens)
    tables = torch.zeros(R, width, dtype=torch.int32)
    dense, qs = [], []
    for r, (c, n) in enumerate(zip(ctx_lens, q_lens)):
        k = torch.randn(c, KV, hd, generator=g)
        v = torch.randn(c, KV, hd, generator=g)
        q = torch.randn(n, H, hd, generator=g)
        if special is not None and special[0] == r:
            u = torch.randn(hd, generator=g)
            u = u / u.norm() * math.sqrt(hd) * 4
            k[special[1]] = u
            q[-1] = u
        k, v, q = (t.to(dtype).float() for t in (k, v, q))
        blocks = [order.pop() for _ in range(-(-c // bs))]
        tables[r, : len(blocks)] = torch.tensor(blocks, dtype=torch.int32)
        for p in range(c):
            kc[blocks[p // bs], :, p % bs] = k[p]
            vc[blocks[p // bs], :, p % bs] = v[p]
        dense.append((k, v))
        qs.append(q)
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    pos_start = torch.tensor([c - n for c, n in zip(ctx_lens, q_lens)], dtype=torch.int32)
    dev = dict(
        q=torch.cat(qs).to(dtype).cuda(), k_cache=kc.to(dtype).cuda(), v_cache=vc.to(dtype).cuda(),
        block_tables=tables.cuda(), req_q_start=q_start.cuda(), req_pos_start=pos_start.cuda(),
    )  # fmt: skip
    return dev, dense, qs


def attention_reference(qs, dense, ctx_lens, q_lens, window):
    outs = []
    for q, (k, v), c, n in zip(qs, dense, ctx_lens, q_lens):
        # run the whole context as queries with zeros in front, keep the last n rows
        full_q = torch.cat([torch.zeros(c - n, *q.shape[1:]), q])
        outs.append(plain.attention(full_q, k, v, window)[c - n :])
    return torch.cat(outs)


ATTN_CASES = [
    # H, KV, hd, bs, ctx_lens, q_lens, window
    (4, 2, 16, 16, [1, 37, 512, 513, 1500], [1, 1, 1, 1, 1], None),
    (32, 8, 128, 16, [700, 33], [1, 33], None),
    (5, 1, 48, 8, [64, 130, 9], [64, 2, 9], None),
    (8, 8, 80, 4, [300, 45], [7, 45], None),
    (6, 3, 32, 8, [200, 77, 24, 25], [1, 30, 24, 2], 24),
    (64, 1, 64, 32, [129], [3], None),
    (16, 8, 256, 16, [90], [90], 17),
    # head sizes 64 and 128: the tensor-core kernels in bfloat16
    (10, 2, 64, 8, [300, 77, 150, 9], [1, 40, 5, 9], None),
    (64, 1, 64, 32, [129, 500], [3, 100], None),
    (32, 8, 128, 16, [2065, 1000, 65], [1, 1, 1], None),
    (16, 4, 128, 16, [600, 200], [600, 8], 100),
    (6, 3, 64, 4, [200, 77, 24, 25], [1, 30, 24, 2], 24),
    (8, 8, 128, 16, [130], [130], None),
    # prompt portions beside single tokens of long requests: the single tokens keep their key partitions
    (8, 2, 128, 16, [2065, 1000, 300, 3000], [1, 1, 200, 1], None),
    (8, 2, 128, 16, [3000, 64, 2500], [1, 64, 3], 700),
    # short rows before, between and after portions, five heads a group: the decode kernel's blocks count short rows only
    (40, 8, 128, 16, [900, 1200, 64, 700, 2100], [2, 300, 1, 8, 1], None),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("case", ATTN_CASES)
def test_paged_attention(ops, dtype, case):
    H, KV, hd, bs, ctx_lens, q_lens, window = case
    dev, dense, qs = paged_setup(ctx_lens, q_lens, H, KV, hd, bs, dtype)
    ref = attention_reference(qs, dense, ctx_lens, q_lens, window)
    common = dict(num_requests=len(ctx_lens), max_context=max(ctx_lens), window=window, scale=hd**-0.5)
    t = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
    parts = (64, (max(ctx_lens) - 1) // 64 + 1)  # the keys split into partitions of 64 and merged
    for generic in (True, False):  # the general kernel, then whichever kernel serving would pick
        out = ops.paged_attention(**dev, **common, generic=generic, host_q_lens=q_lens)
        assert torch.allclose(out.float().cpu(), ref, **t), f"generic={generic}"
        if generic or max(q_lens) <= 8 or (dtype == torch.bfloat16 and hd == 128 and min(q_lens) <= 8):
            out2 = ops.paged_attention(**dev, **common, generic=generic, host_q_lens=q_lens, partitions=parts)
            assert torch.allclose(out2.float().cpu(), ref, **t), f"generic={generic} partitioned"
    out3 = ops.paged_attention(**dev, **common)  # without host knowledge of the portions
    assert torch.allclose(out3.float().cpu(), ref, **t)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("where", [0, 15, 16, 17, 255, 256, 511, 640, 999])
def test_attention_finds_one_far_key(ops, dtype, where):
    """One key among a thousand matches the query strongly: the output must be its value,
    wherever in its page and partition it lies."""
    H, KV, hd, bs, ctx = 8, 2, 64, 16, 1000
    dev, dense, qs = paged_setup([ctx], [1], H, KV, hd, bs, dtype, seed=where, special=(0, where))
    for parts, generic in ((None, False), ((256, 4), False), (None, True), ((256, 4), True)):
        out = ops.paged_attention(**dev, num_requests=1, max_context=ctx, window=None, scale=hd**-0.5,
                                  partitions=parts, generic=generic, host_q_lens=[1])  # fmt: skip
        v = dense[0][1][where]  # [KV, hd]
        expect = v.repeat_interleave(H // KV, dim=0)
        assert torch.allclose(out[0].float().cpu(), expect, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_window_edge(ops, dtype):
    """The key at p - window + 1 is seen, the key at p - window is not."""
    for hd in (32, 64):
        H, KV, bs, ctx, window = 4, 2, 8, 120, 24
        p = ctx - 1
        for where, seen in ((p - window + 1, True), (p - window, False)):
            for n in (1, 12):  # as a single decoded token, and as the last row of a portion
                dev, dense, qs = paged_setup([ctx], [n], H, KV, hd, bs, dtype, seed=3, special=(0, where))
                out = ops.paged_attention(**dev, num_requests=1, max_context=ctx, window=window, scale=hd**-0.5,
                                          host_q_lens=[n])  # fmt: skip
                expect = dense[0][1][where].repeat_interleave(H // KV, dim=0)
                close = torch.allclose(out[-1].float().cpu(), expect, atol=2e-2, rtol=2e-2)
                assert close == seen, (hd, where, n)


@pytest.mark.parametrize("prefill_kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("window", [100, 108])
def test_attention_window_edge_head_128(ops, monkeypatch, prefill_kernel, window):
    """The served head size, through the tensor-core kernels: a single decoded token (the mma
    decode kernel), the last row of a short portion and of a 200-token portion (the tcgen05
    kernel, then the mma prefill kernel). With 300 keys the window of 100 begins at key 200, inside
    a 64-key tile and inside a page; the window of 108 begins at key 192, the first key of a tile
    and of a page, so the unseen key is the last of the tile and page before."""
    import atomserve_b200.ops.attention as A

    monkeypatch.setattr(A, "PREFILL_KERNEL", prefill_kernel)
    H, KV, hd, bs, ctx = 8, 2, 128, 16, 300
    p = ctx - 1
    for where, seen in ((p - window + 1, True), (p - window, False)):
        for n in (1, 12, 200):
            dev, dense, qs = paged_setup([ctx], [n], H, KV, hd, bs, torch.bfloat16, seed=5, special=(0, where))
            out = ops.paged_attention(**dev, num_requests=1, max_context=ctx, window=window, scale=hd**-0.5,
                                      host_q_lens=[n])  # fmt: skip
            expect = dense[0][1][where].repeat_interleave(H // KV, dim=0)
            close = torch.allclose(out[-1].float().cpu(), expect, atol=2e-2, rtol=2e-2)
            assert close == seen, (prefill_kernel, window, where, n)
            ref = attention_reference(qs, dense, [ctx], [n], window)  # and every other row of the portion
            assert torch.allclose(out.float().cpu(), ref, atol=2e-2, rtol=2e-2), (prefill_kernel, window, where, n)
    from atomserve_b200.ops.linear import check_gemm_status

    check_gemm_status()


def long_context_setup(ctx_lens, q_lens, H, KV, hd, bs, seed, special=None):
    """Long requests without per-position Python loops: one pool of random pages on the device,
    shared by all requests, each request reading it through a shuffled block table of its own (so
    every request sees other keys in another order). Returns the device inputs and, per request,
    its keys and values in position order as float32 on the CPU. `special` = (request, position):
    that key matches the request's last query strongly."""
    g = torch.Generator().manual_seed(seed)
    pages = max(-(-c // bs) for c in ctx_lens)
    pool = pages + 5
    kc = (torch.randn(pool, KV, bs, hd, generator=g) * 0.5).bfloat16()
    vc = torch.randn(pool, KV, bs, hd, generator=g).bfloat16()
    tables = torch.stack([torch.randperm(pool, generator=g)[:pages] for _ in ctx_lens]).to(torch.int32)
    q = torch.randn(sum(q_lens), H, hd, generator=g).bfloat16()
    q_start = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32)
    if special is not None:
        r, where = special
        u = torch.randn(hd, generator=g)
        u = (u / u.norm() * math.sqrt(hd) * 4).bfloat16()
        kc[tables[r, where // bs], :, where % bs] = u
        q[int(q_start[r + 1]) - 1] = u
    dense = []
    for r, c in enumerate(ctx_lens):
        mine = tables[r].long()
        k = kc[mine].permute(0, 2, 1, 3).reshape(-1, KV, hd)[:c].float()
        v = vc[mine].permute(0, 2, 1, 3).reshape(-1, KV, hd)[:c].float()
        dense.append((k, v))
    pos_start = torch.tensor([c - n for c, n in zip(ctx_lens, q_lens)], dtype=torch.int32)
    dev = dict(q=q.cuda(), k_cache=kc.cuda(), v_cache=vc.cuda(), block_tables=tables.cuda(),
               req_q_start=q_start.cuda(), req_pos_start=pos_start.cuda())  # fmt: skip
    return dev, dense, q.float()


def long_context_reference(q, dense, ctx_lens, q_lens, window=None):
    outs, at = [], 0
    for (k, v), c, n in zip(dense, ctx_lens, q_lens):
        outs.append(plain.attention_rows(q[at : at + n], k, v, torch.arange(c - n, c), window))
        at += n
    return torch.cat(outs)


@pytest.mark.parametrize("context", [8192, 32768])
@pytest.mark.parametrize("batch", [1, 8, 64])
def test_decode_attention_at_long_contexts(ops, batch, context):
    """Single decoded tokens over 8k and 32k keys with the key partitions that the planner picks
    for 1, 8 and 64 requests, against the plain attention; the requests' contexts differ, the
    longest being `context`, and in request 0 one far key carries nearly all the weight."""
    from atomserve_b200.ops.attention import plan_decode_partitions

    H, KV, hd, bs = 8, 2, 128, 16
    ctx_lens = [context - (37 * r) % (context // 2) for r in range(batch)]
    where = context // 3 + 5
    dev, dense, q = long_context_setup(ctx_lens, [1] * batch, H, KV, hd, bs, seed=batch, special=(0, where))
    size, parts = plan_decode_partitions(batch, KV, H // KV, context, 0, hd)
    assert parts > 1 and size * parts >= context and size % 64 == 0
    out = ops.paged_attention(**dev, num_requests=batch, max_context=context, window=None, scale=hd**-0.5,
                              host_q_lens=[1] * batch).float().cpu()  # fmt: skip
    ref = long_context_reference(q, dense, ctx_lens, [1] * batch)
    assert torch.allclose(out, ref, atol=2e-2, rtol=2e-2), float((out - ref).abs().max())
    expect = dense[0][1][where].repeat_interleave(H // KV, dim=0)
    assert torch.allclose(out[0], expect, atol=2e-2, rtol=2e-2)
    general = ops.paged_attention(**dev, num_requests=batch, max_context=context, window=None, scale=hd**-0.5,
                                  host_q_lens=[1] * batch, generic=True).float().cpu()  # fmt: skip
    assert torch.allclose(general, ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("prefill_kernel", ["tcgen05", "mma"])
@pytest.mark.parametrize("ctx,n", [(8192, 8192), (8192, 512)])
def test_prefill_attention_at_long_contexts(ops, monkeypatch, prefill_kernel, ctx, n):
    """One prompt of 8,192 tokens in one step, and a portion of 512 tokens behind 7,680 cached
    ones, against the plain attention row by row."""
    import atomserve_b200.ops.attention as A
    from atomserve_b200.ops.linear import check_gemm_status

    monkeypatch.setattr(A, "PREFILL_KERNEL", prefill_kernel)
    H, KV, hd, bs = 4, 1, 128, 16
    dev, dense, q = long_context_setup([ctx], [n], H, KV, hd, bs, seed=n, special=(0, 100))
    out = ops.paged_attention(**dev, num_requests=1, max_context=ctx, window=None, scale=hd**-0.5,
                              host_q_lens=[n]).float().cpu()  # fmt: skip
    check_gemm_status()
    ref = long_context_reference(q, dense, [ctx], [n])
    assert torch.allclose(out, ref, atol=2e-2, rtol=2e-2), float((out - ref).abs().max())
    assert torch.allclose(out[-1], dense[0][1][100].repeat_interleave(H // KV, dim=0), atol=2e-2, rtol=2e-2)


def test_sampling_greedy_and_support(ops):
    logits = torch.tensor([[0.1, 3.0, 0.2, 3.0], [5.0, 1.0, 0.0, -1.0]], device="cuda")
    assert ops.argmax_rows(logits).tolist() == [1, 0]  # lowest id among equals

    probs = torch.tensor([0.4, 0.3, 0.2, 0.1])

    def draws(n, temperature, top_k, top_p, seed=1):
        lg = probs.log().repeat(n, 1).cuda().contiguous()
        return ops.sample_rows(
            lg, torch.full((n,), temperature, device="cuda"), torch.full((n,), top_k, dtype=torch.int32, device="cuda"),
            torch.full((n,), top_p, device="cuda"), torch.full((n,), seed, dtype=torch.int64, device="cuda"),
            torch.arange(n, dtype=torch.int64, device="cuda"),
        ).cpu()  # fmt: skip

    counts = draws(20000, 1.0, 0, 1.0).bincount(minlength=4)
    assert torch.allclose(counts / 20000, probs, atol=0.015)
    assert set(draws(2000, 1.0, 2, 1.0).tolist()) == {0, 1}
    assert set(draws(200, 1.0, 1, 1.0).tolist()) == {0}
    assert set(draws(2000, 1.0, 0, 0.6).tolist()) == {0, 1}
    assert set(draws(200, 1.0, 0, 0.01).tolist()) == {0}
    assert set(draws(50, 0.0, 3, 0.5).tolist()) == {0}
    # temperature reshapes the distribution: p^(1/T) renormalised
    counts = draws(20000, 0.5, 0, 1.0).bincount(minlength=4)
    sharp = probs**2 / (probs**2).sum()
    assert torch.allclose(counts / 20000, sharp, atol=0.015)


@pytest.mark.parametrize("V,k,p,temp", [(331, 20, 0.95, 0.6), (5000, 64, 0.8, 0.7), (151936, 20, 0.95, 0.6),
                                        (2000, 0, 0.9, 1.0), (3000, 1500, 0.5, 1.3)])  # fmt: skip
def test_sampling_support_matches_plain(ops, V, k, p, temp):
    """Everything drawn lies in the plain sampler's support, and frequent tokens agree."""
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(V, generator=g) * 3
    dist = plain.sampling_distribution(logits, temp, k, p)
    n = 4000
    out = ops.sample_rows(
        logits.repeat(n, 1).cuda().contiguous(), torch.full((n,), temp, device="cuda"),
        torch.full((n,), k, dtype=torch.int32, device="cuda"), torch.full((n,), p, device="cuda"),
        torch.full((n,), 9, dtype=torch.int64, device="cuda"), torch.arange(n, dtype=torch.int64, device="cuda"),
    ).cpu().long()  # fmt: skip
    assert bool((dist[out] > 0).all())
    freq = out.bincount(minlength=V) / n
    assert float((freq - dist).abs().max()) < 0.04


def test_sampling_ties_at_the_cut(ops):
    """Equal logits at the k-th place: exactly k tokens stay, the lower ids."""
    logits = torch.tensor([[1.0, 2.0, 2.0, 2.0, 2.0, 0.5, 3.0]], device="cuda").repeat(500, 1).contiguous()
    n = 500
    out = ops.sample_rows(
        logits, torch.ones(n, device="cuda"), torch.full((n,), 3, dtype=torch.int32, device="cuda"),
        torch.ones(n, device="cuda"), torch.zeros(n, dtype=torch.int64, device="cuda"),
        torch.arange(n, dtype=torch.int64, device="cuda"),
    ).cpu()  # fmt: skip
    assert set(out.tolist()) == {6, 1, 2}


def test_seeded_rows_do_not_depend_on_neighbours(ops):
    g = torch.Generator().manual_seed(0)
    row = torch.randn(1000, generator=g)
    others = torch.randn(2, 1000, generator=g)

    def run(rows, seeds, counters):
        n = rows.shape[0]
        return ops.sample_rows(
            rows.cuda().contiguous(), torch.ones(n, device="cuda"), torch.full((n,), 50, dtype=torch.int32, device="cuda"),
            torch.ones(n, device="cuda"), torch.tensor(seeds, dtype=torch.int64, device="cuda"),
            torch.tensor(counters, dtype=torch.int64, device="cuda"),
        ).tolist()  # fmt: skip

    alone = [run(row[None], [7], [i])[0] for i in range(20)]
    crowd = [run(torch.stack([others[0], row, others[1]]), [1, 7, 2], [i + 5, i, i + 9])[1] for i in range(20)]
    assert alone == crowd and len(set(alone)) > 3


def test_presence_penalty(ops):
    logits = torch.zeros(2, 10, device="cuda")
    ops.presence_penalty(
        logits, torch.tensor([0, 0, 1], dtype=torch.int32, device="cuda"),
        torch.tensor([3, 4, 9], dtype=torch.int32, device="cuda"), torch.tensor([1.5, 1.5, 0.5], device="cuda"),
    )  # fmt: skip
    expect = torch.zeros(2, 10)
    expect[0, 3] = expect[0, 4] = -1.5
    expect[1, 9] = -0.5
    assert torch.equal(logits.cpu(), expect)


GEMM_SHAPES = [
    (1, 128, 64), (3, 100, 72), (16, 256, 512), (17, 384, 4096), (33, 130, 1024), (64, 4096, 4096),
    (8, 4096, 12288), (65, 256, 128), (128, 300, 264), (300, 512, 1000), (2048, 1024, 512),
    (200, 4096, 1024), (256, 512, 2048), (100, 24576, 256), (40, 20000, 128),
    (300, 4096, 512), (512, 4104, 256), (700, 5120, 128), (384, 6144, 192),
    (300, 4096, 8192), (512, 1000, 8256), (257, 2048, 12288),
]  # fmt: skip


@pytest.mark.parametrize("M,N,K", GEMM_SHAPES)
def test_gemm_tcgen05(ops, M, N, K):
    """The tcgen05/TMEM/TMA GEMM against float64, in every epilogue, swapped and split shapes
    included; its status word must stay zero (no pipeline wait ran out)."""
    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05

    g = torch.Generator().manual_seed(M * 7 + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    res = torch.randn(M, N, generator=g).bfloat16().cuda()
    ref = x.double().cpu() @ w.double().cpu().T
    full = gemm_tcgen05(x, w, None, torch.float32)
    check_gemm_status()
    assert torch.allclose(full.double().cpu(), ref, atol=2e-3, rtol=1e-3), float((full.double().cpu() - ref).abs().max())
    plain_out = gemm_tcgen05(x, w, None, torch.bfloat16)
    with_res = gemm_tcgen05(x, w, res, torch.bfloat16)
    check_gemm_status()
    assert torch.allclose(plain_out.double().cpu(), ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(with_res.double().cpu(), ref + res.double().cpu(), atol=3e-2, rtol=2e-2)
    # a row's result does not depend on the rows beside it (same kernel shape: same tile path)
    if M > 1:
        again = gemm_tcgen05(x, w, None, torch.float32)
        assert torch.equal(again, full)


TCGEN05_ATTN_CASES = [
    # H, KV, bs, ctx_lens, q_lens, window
    (4, 1, 16, [200], [200], None),
    (32, 8, 16, [700, 33, 2100], [1, 33, 300], None),
    (8, 8, 8, [130, 500], [130, 260], None),
    (16, 8, 32, [640, 129, 77], [129, 129, 9], None),
    (16, 2, 64, [1000], [333], 200),
    (16, 1, 128, [300, 150], [100, 150], 64),
    (8, 2, 16, [2048], [2048], None),
    # groups that do not divide 128: 25, 42 and 18 tokens a tile, the last rows of a tile padding
    (40, 8, 16, [700, 90, 300], [300, 90, 1], None),
    (6, 2, 16, [500], [500], 130),
    (7, 1, 32, [333, 64], [200, 64], None),
]


@pytest.mark.parametrize("case", TCGEN05_ATTN_CASES)
def test_prefill_attention_tcgen05(ops, case):
    """The tcgen05 prefill kernel (scores and output in tensor memory, V as an MN-major operand,
    pages fetched by TMA) against the plain attention, and against the mma.sync kernel it
    replaces; prompt portions with a cached prefix, several requests, windows, every group size
    and page size it serves."""
    from atomserve_b200.ops import attention as attn
    from atomserve_b200.ops.linear import check_gemm_status

    H, KV, bs, ctx_lens, q_lens, window = case
    hd = 128
    dev, dense, qs = paged_setup(ctx_lens, q_lens, H, KV, hd, bs, torch.bfloat16, seed=H + bs)
    ref = attention_reference(qs, dense, ctx_lens, q_lens, window)
    common = dict(num_requests=len(ctx_lens), max_context=max(ctx_lens), window=window, scale=hd**-0.5, host_q_lens=q_lens)
    assert attn.lib().asb_attention_tcgen05_supported(hd, H // KV, bs)
    results = {}
    for kernel in ("tcgen05", "mma"):
        attn.PREFILL_KERNEL = kernel
        try:
            results[kernel] = ops.paged_attention(**dev, **common).float().cpu()
        finally:
            attn.PREFILL_KERNEL = "tcgen05"
    check_gemm_status()
    assert torch.allclose(results["tcgen05"], ref, atol=2e-2, rtol=2e-2), float((results["tcgen05"] - ref).abs().max())
    assert torch.allclose(results["mma"], ref, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("M,I,K", [(1, 64, 64), (5, 200, 72), (16, 1024, 512), (40, 352, 256), (64, 12288, 4096),
                                   (100, 176, 80), (300, 704, 256), (2048, 512, 512)])  # fmt: skip
def test_gemm_tcgen05_swiglu(ops, M, I, K):
    """silu(x gate^T) * (x up^T) from the GEMM's own epilogue (and, where K is cut, from the
    reduction of its partial sums) against float64."""
    from atomserve_b200.ops.linear import check_gemm_status

    g = torch.Generator().manual_seed(M + I + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    gate = (torch.randn(I, K, generator=g) / math.sqrt(K) * 2).bfloat16().cuda()
    up = (torch.randn(I, K, generator=g) / math.sqrt(K) * 2).bfloat16().cuda()
    w = ops.interleave_gate_up(gate, up)
    assert torch.equal(w[0::2], gate) and torch.equal(w[1::2], up)
    if not ops.swiglu_fusable(w):
        pytest.skip("the tensor-core GEMM is switched off (ATOMSERVE_B200_GEMM)")
    out = ops.linear_swiglu(x, w)
    check_gemm_status()
    gs, us = x.double().cpu() @ gate.double().cpu().T, x.double().cpu() @ up.double().cpu().T
    ref = gs / (1 + torch.exp(-gs)) * us
    assert out.shape == (M, I) and torch.allclose(out.double().cpu(), ref, atol=2e-2, rtol=2e-2)


def _skip_without_partial_sums():
    import importlib

    L = importlib.import_module("atomserve_b200.ops.linear")
    if not L.PARTIAL_SUMS or L.BACKEND != "tcgen05":
        pytest.skip("partial sums are switched off (ATOMSERVE_B200_PARTIAL_SUMS, ATOMSERVE_B200_GEMM)")


PARTIAL_NORM_SHAPES = [(1, 4096, 4096), (8, 4096, 12288), (5, 1024, 2048), (16, 640, 1024), (33, 2048, 4096),
                       (64, 4096, 4096), (7, 5120, 17408), (3, 264, 2048), (100, 4096, 4096), (128, 1024, 2048)]  # fmt: skip


@pytest.mark.parametrize("M,N,K", PARTIAL_NORM_SHAPES)
def test_partial_add_rms_norm_is_the_unfused_result(ops, M, N, K):
    """A product left as the GEMM's partial sums, added up with the residual and normalised in
    one kernel: the same bits as the GEMM with its own reduction followed by rms_norm, and close
    to float64."""
    from atomserve_b200.ops.linear import check_gemm_status

    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    res = torch.randn(M, N, generator=g).bfloat16().cuda()
    gain = (1 + 0.1 * torch.randn(N, generator=g)).cuda()
    _skip_without_partial_sums()
    product = ops.linear_partial(x, w)
    assert product is not None, "these shapes cut K: the partial-sum form must be available"
    assert (product.tokens, product.columns) == (M, N)
    total, normed = ops.partial_add_rms_norm(product, res, gain, 1e-6)
    plain_total = ops.linear(x, w, res)
    plain_normed = ops.rms_norm(plain_total, gain, 1e-6)
    check_gemm_status()
    assert torch.equal(total, plain_total) and torch.equal(normed, plain_normed)
    ref = x.double().cpu() @ w.double().cpu().T + res.double().cpu()
    assert torch.allclose(total.double().cpu(), ref, atol=3e-2, rtol=2e-2)
    # without a residual
    total0, normed0 = ops.partial_add_rms_norm(ops.linear_partial(x, w), None, gain, 1e-6)
    plain0 = ops.linear(x, w)
    assert torch.equal(total0, plain0) and torch.equal(normed0, ops.rms_norm(plain0, gain, 1e-6))


def test_linear_partial_declines_what_does_not_cut_k(ops):
    """Many tokens, float32 operands and tiny products have no partial-sum form: None, and the
    caller takes the plain product."""
    x = torch.randn(300, 512, device="cuda").bfloat16()
    w = torch.randn(1024, 512, device="cuda").bfloat16()
    assert ops.linear_partial(x, w) is None
    assert ops.linear_partial(x[:4].float(), w.float()) is None


# beyond 128 tokens the planner rarely swaps the operands and cuts K (which is when the product can
# be left as partial sums): the last shape's 150 tokens run with that form forced
QKV_PARTIAL_SHAPES = [(8, 2, 128, 2048), (32, 8, 128, 4096), (4, 2, 64, 1024), (6, 3, 32, 2048), (2, 1, 256, 1024), (8, 0, 128, 2048),
                      (4, 1, 128, 12288)]  # fmt: skip


@pytest.mark.parametrize("T,H,KV,hd,K", [(T, *shape) for shape in QKV_PARTIAL_SHAPES for T in (1, 6, 40, 128, 150)
                                         if T <= 128 or shape[3] >= 12288])  # fmt: skip
def test_qk_norm_rope_store_from_partial_sums(ops, T, H, KV, hd, K):
    """q/k norm, rotation and the cache write reading the qkv product from the GEMM's partial
    sums: the same bits as from the reduced product (KV = 0: queries only, nothing stored)."""
    from atomserve_b200.ops.linear import check_gemm_status, gemm_tune

    _skip_without_partial_sums()
    g = torch.Generator().manual_seed(H * 100 + hd + T)
    bs, nblocks = 16, 12
    x = torch.randn(T, K, generator=g).bfloat16().cuda()
    w = (torch.randn((H + 2 * KV) * hd, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    qg, kg = ((1 + 0.1 * torch.randn(hd, generator=g)).cuda() for _ in range(2))
    inv_freq = plain.rope_inv_freq(hd, 1e6).cuda()
    pos = torch.randint(0, 40000, (T,), generator=g).int().cuda()
    slot_list = torch.randperm(nblocks * bs, generator=g)[:T].tolist()
    if T > 1:
        slot_list[1] = -1
    slots = torch.tensor(slot_list, dtype=torch.int32, device="cuda")
    results = []
    for partial in (False, True):
        kc = torch.zeros(nblocks, max(KV, 1), bs, hd, device="cuda", dtype=torch.bfloat16)
        vc = torch.zeros_like(kc)
        if T > 128:
            gemm_tune(1)  # swapped operands: tiles of 128 weight rows by 256 tokens
        try:
            qkv = ops.linear_partial(x, w) if partial else ops.linear(x, w)
        finally:
            gemm_tune()
        assert qkv is not None
        store = dict(slots=slots, k_cache=kc, v_cache=vc) if KV else dict(slots=None, k_cache=None, v_cache=None)
        q = ops.qk_norm_rope_store(qkv, H, KV, hd, pos, q_gain=qg, k_gain=kg, eps=1e-6, inv_freq=inv_freq,
                                   rotary_dim=hd, **store)  # fmt: skip
        results.append((q, kc, vc))
    check_gemm_status()
    for a, b in zip(*results):
        assert torch.equal(a, b)
    assert float(results[1][0].float().abs().max()) > 0


def test_captured_gemm_survives_workspace_growth(ops):
    """A CUDA graph captured while the GEMM's partial-sum workspace was small keeps working after
    a larger call has replaced it: the outgrown buffer stays alive for the graphs that use it."""
    import importlib

    L = importlib.import_module("atomserve_b200.ops.linear")  # `ops.linear` itself is the function
    g = torch.Generator().manual_seed(5)
    x = torch.randn(8, 4096, generator=g).bfloat16().cuda()
    w = (torch.randn(4096, 4096, generator=g) / 64).bfloat16().cuda()
    expect = L.gemm_tcgen05(x, w, None, torch.bfloat16).clone()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = L.gemm_tcgen05(x, w, None, torch.bfloat16)
    before = L.gemm_workspace(x.device, 1)
    L.gemm_workspace(x.device, before.numel() + 1)  # a larger call comes along
    assert L.gemm_workspace(x.device, 1) is not before
    junk = [torch.full((before.numel(),), float("nan"), device="cuda") for _ in range(2)]  # would land in freed memory
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, expect)
    del junk
    L.check_gemm_status()


def test_a_wait_that_runs_out_reports_frees_tensor_memory_and_returns(ops):
    """The give-up path of the tcgen05 kernels, executed on purpose by a kernel that waits (a few
    thousand polls) on a barrier nothing arrives at: the status word names it, the block frees its
    tensor memory and ends, the context stays usable, and a GEMM that needs all of an SM's tensor
    memory runs right afterwards. The engine's step would fail with this report."""
    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05
    from atomserve_b200.ops.status import bounded_wait_selftest, status_for

    check_gemm_status()
    for _ in range(3):  # repeatedly: tensor memory that was not freed would run out or stall
        report = bounded_wait_selftest("cuda", polls=2048)
        assert report is not None and "self-test" in report and "gave up a bounded wait" in report
    assert status_for("cuda").problem() is None  # cleared by the read
    x = torch.randn(128, 512, device="cuda").bfloat16()
    w = torch.randn(384, 512, device="cuda").bfloat16()
    out = gemm_tcgen05(x, w, None, torch.float32)
    check_gemm_status()
    assert torch.allclose(out.double().cpu(), x.double().cpu() @ w.double().cpu().T, atol=2e-2, rtol=1e-3)


# the last three leave a last round of few tiles, which the kernel cuts along K (for one or both tile widths)
PAIR_SHAPES = [(300, 512, 256), (257, 1000, 520), (129, 130, 72), (2048, 4096, 4096), (700, 6144, 4160),
               (513, 24576, 1024), (1000, 256, 64), (3000, 384, 200), (640, 4104, 8),
               (1000, 5000, 4160), (300, 4000, 4160), (520, 1100, 2120)]  # fmt: skip


@pytest.mark.parametrize("rows", [128, 160, 224, 256])
@pytest.mark.parametrize("M,N,K", PAIR_SHAPES)
def test_gemm_tcgen05_on_pairs_of_sms(ops, M, N, K, rows):
    """The many-token form of the GEMM (tcgen05.mma.cta_group::2: two CTAs on a tile of 256 tokens
    by 128 to 256 weight rows), forced for shapes the planner would also give to single SMs: every
    epilogue against float64; tokens, weight rows and K that end inside a tile, an odd number of K
    blocks (the second K block of the last stage lies beyond K), one tile, many tiles per pair, a
    last round of tiles cut along K into pieces that a second kernel adds up."""
    from atomserve_b200.ops.linear import check_gemm_status, gemm_tcgen05, gemm_tune

    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).bfloat16().cuda()
    w = (torch.randn(N, K, generator=g) / math.sqrt(K)).bfloat16().cuda()
    res = torch.randn(M, N, generator=g).bfloat16().cuda()
    ref = x.double().cpu() @ w.double().cpu().T
    gemm_tune(2, rows)
    try:
        full = gemm_tcgen05(x, w, None, torch.float32)
        plain_out = gemm_tcgen05(x, w, None, torch.bfloat16)
        with_res = gemm_tcgen05(x, w, res, torch.bfloat16)
        fused = gemm_tcgen05(x, w, None, torch.bfloat16, swiglu=True) if N % 2 == 0 else None
        again = gemm_tcgen05(x, w, None, torch.float32)
        gemm_tune(2, rows, cut_last_round=False)
        uncut = gemm_tcgen05(x, w, None, torch.float32)
    finally:
        gemm_tune()
    check_gemm_status()
    # cut or whole, the same products are added, in another order
    assert torch.allclose(uncut, full, atol=1e-4, rtol=1e-4)
    assert torch.allclose(full.double().cpu(), ref, atol=2e-3, rtol=1e-3), float((full.double().cpu() - ref).abs().max())
    assert torch.equal(again, full)
    assert torch.allclose(plain_out.double().cpu(), ref, atol=3e-2, rtol=2e-2)
    assert torch.allclose(with_res.double().cpu(), ref + res.double().cpu(), atol=3e-2, rtol=2e-2)
    if fused is not None:
        gate, up = ref[:, 0::2], ref[:, 1::2]
        assert torch.allclose(fused.double().cpu(), gate / (1 + torch.exp(-gate)) * up, atol=3e-2, rtol=3e-2)
