"""The allocation-free attention entry point, called through its exported C symbol.

Some hosts of these kernels cannot allocate device memory around a call: the process gave the
GPU's memory away at start-up, or it cannot afford cudaMalloc's synchronisation, or it is a
foreign runtime with only raw pointers to offer. For them the library exports
`asb_paged_attention_static_scratch`, which keeps the split-key partial results in an array of
its own (atomserve_b200/csrc/attention_noalloc.h). This test calls it twice in a row on
different inputs and compares each result with the ordinary entry point's, which takes its
scratch from the caller. The file is named to be collected last, so that a run which stops at
the first failure has run every other test before it.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


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
        tol = dict(atol=2e-5, rtol=1e-4) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)
        assert torch.allclose(out.float(), expect.float(), **tol)


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
