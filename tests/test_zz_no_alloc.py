"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of these kernels cannot allocate device memory around a call: the process gave the
GPU's memory away at start-up, or it cannot afford cudaMalloc's synchronisation, or it is a
foreign runtime with only raw pointers to offer. For them the library exports
`asb_paged_attention_static_scratch`, which keeps the split-key partial results in an array of
its own (atomserve_b200/csrc/attention_noalloc.h). This test calls it twice in a row on
different inputs and holds each result to two things: the ordinary entry point's result, which
takes its scratch from the caller and must agree bit for bit (same kernels, same order of
additions), and the plain attention of tests/plain_qwen3.py on the gathered keys and values.
A call that needs no partitions must go through however many tokens it brings. The file is named
to be collected last, so that a run which stops at the first failure has run every other test
before it.
"""

import ctypes

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu


def plain_decode_attention(q, kc, vc, tables, ctx_lens, bs):
    """Each request's last-position output by the plain implementation: its keys and values
    gathered from the pages in position order, the query placed at the last position."""
    outs = []
    for r, n in enumerate(ctx_lens):
        pages = tables[r, : -(-n // bs)].long().cpu()
        k = kc.float().cpu()[pages].permute(0, 2, 1, 3).reshape(-1, kc.shape[1], kc.shape[3])[:n]
        v = vc.float().cpu()[pages].permute(0, 2, 1, 3).reshape(-1, vc.shape[1], vc.shape[3])[:n]
        qq = torch.zeros(n, q.shape[1], q.shape[2])
        qq[-1] = q[r].float().cpu()
        outs.append(plain.attention(qq, k, v)[-1])
    return torch.stack(outs)


def entry_point():
    from atomserve_b200.ops import library

    handle = library.lib()
    fn = handle.asb_paged_attention_static_scratch
    p, i = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [p] * 7 + [i] * 10 + [ctypes.c_float, i, p]
    fn.restype = i
    handle.asb_static_scratch_floats.restype = ctypes.c_uint
    return handle, fn


def make_inputs(seed, dtype, ctx_lens, H=8, KV=2, hd=64, bs=16):
    g = torch.Generator().manual_seed(seed)
    R = len(ctx_lens)
    width = max(-(-c // bs) for c in ctx_lens)
    nblocks = R * width + 2
    order = torch.randperm(nblocks, generator=g)
    tables = order[: R * width].reshape(R, width).to(torch.int32).cuda()
    kc = torch.randn(nblocks, KV, bs, hd, generator=g).to(dtype).cuda()
    vc = torch.randn(nblocks, KV, bs, hd, generator=g).to(dtype).cuda()
    q = torch.randn(R, H, hd, generator=g).to(dtype).cuda()
    q_start = torch.arange(R + 1, dtype=torch.int32).cuda()
    pos_start = torch.tensor([c - 1 for c in ctx_lens], dtype=torch.int32).cuda()
    return q, kc, vc, tables, q_start, pos_start


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_static_scratch_entry_point_matches_the_allocating_one(dtype):
    from atomserve_b200 import ops
    from atomserve_b200.ops.library import dtype_code

    handle, fn = entry_point()
    H, KV, hd, bs, PS = 8, 2, 64, 16, 64
    for call, ctx_lens in enumerate(([300, 17, 129], [64, 511])):  # two calls in a row share the array
        q, kc, vc, tables, q_start, pos_start = make_inputs(call, dtype, ctx_lens)
        NP = (max(ctx_lens) - 1) // PS + 1
        expect = ops.paged_attention(q, kc, vc, tables, q_start, pos_start, num_requests=len(ctx_lens),
                                     max_context=max(ctx_lens), window=None, scale=hd**-0.5,
                                     partitions=(PS, NP), generic=True)  # fmt: skip
        out = torch.empty_like(q)
        rc = fn(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), q_start.data_ptr(),
                pos_start.data_ptr(), q.shape[0], len(ctx_lens), H, KV, hd, bs, tables.shape[1], 0, PS, NP,
                hd**-0.5, dtype_code(q), torch.cuda.current_stream().cuda_stream)  # fmt: skip
        assert rc == 0, handle.asb_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(out, expect)  # the same kernels on other scratch: the same bits
        tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        oracle = plain_decode_attention(q, kc, vc, tables, ctx_lens, bs)
        assert torch.allclose(out.float().cpu(), oracle, **tol)


def test_static_scratch_is_not_asked_of_a_call_without_partitions():
    """2,048 tokens of 32 heads would need 8.5 Mi floats if they were partitioned; with one
    partition the kernel writes its output directly, so the call must pass."""
    from atomserve_b200 import ops
    from atomserve_b200.ops.library import dtype_code

    handle, fn = entry_point()
    H, KV, hd, bs, T = 32, 8, 64, 16, 2048
    g = torch.Generator().manual_seed(3)
    pages = T // bs
    tables = torch.randperm(pages + 3, generator=g)[:pages].reshape(1, pages).to(torch.int32).cuda()
    kc = torch.randn(pages + 3, KV, bs, hd, generator=g).cuda()
    vc = torch.randn(pages + 3, KV, bs, hd, generator=g).cuda()
    q = torch.randn(T, H, hd, generator=g).cuda()
    q_start = torch.tensor([0, T], dtype=torch.int32).cuda()
    pos_start = torch.zeros(1, dtype=torch.int32).cuda()
    assert T * H * (hd + 2) > handle.asb_static_scratch_floats()
    expect = ops.paged_attention(q, kc, vc, tables, q_start, pos_start, num_requests=1, max_context=T, window=None,
                                 scale=hd**-0.5, partitions=(1 << 30, 1), generic=True)  # fmt: skip
    out = torch.empty_like(q)
    rc = fn(out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), q_start.data_ptr(),
            pos_start.data_ptr(), T, 1, H, KV, hd, bs, pages, 0, 1 << 30, 1, hd**-0.5, dtype_code(q),
            torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert rc == 0, handle.asb_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(out, expect)


def test_static_scratch_refuses_what_does_not_fit():
    handle, fn = entry_point()
    capacity = handle.asb_static_scratch_floats()
    assert capacity == 4 * 1024 * 1024
    q, kc, vc, tables, q_start, pos_start = make_inputs(0, torch.float32, [40])
    tokens, H, hd, NP = 4096, 32, 128, 9  # 4096 * 32 * 9 * 130 floats: far beyond the array
    rc = fn(None, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), q_start.data_ptr(),
            pos_start.data_ptr(), tokens, 1, H, 2, hd, 16, tables.shape[1], 0, 64, NP, 1.0, 0,
            torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert rc != 0
    message = handle.asb_last_error().decode()
    assert "exceed the built-in scratch" in message and str(capacity) in message
    # numbers whose product would wrap 64 bits are refused by range, not by a wrapped product
    rc = fn(None, q.data_ptr(), kc.data_ptr(), vc.data_ptr(), tables.data_ptr(), q_start.data_ptr(),
            pos_start.data_ptr(), 2**31 - 1, 1, 2**31 - 1, 2, hd, 16, tables.shape[1], 0, 64, 2**31 - 1, 1.0, 0,
            torch.cuda.current_stream().cuda_stream)  # fmt: skip
    assert rc != 0 and "out of range" in handle.asb_last_error().decode()
