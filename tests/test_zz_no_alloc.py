"""All-reduce for callers that must not allocate device memory.

``tccl_allreduce_sum_noalloc`` sums buffers that live on one GPU using scratch
memory built into the library image, so a caller whose memory is handed out once
and then frozen (a fixed pool, a latency-critical loop, a plug-in that only gets
buffers from its host) never triggers cudaMalloc.  The test drives it through its
exported C symbol and compares with the library's ordinary heap-based all-reduce
on the same data, twice in a row (the second call reuses the scratch the first one
left behind).  This file sorts last on purpose: a run that stops at the first
failure has then already run every other test.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

DTYPES = {torch.float16: (0, 2e-2), torch.bfloat16: (1, 2e-2), torch.float32: (2, 1e-5)}


def _symbol():
    from tileccl_b200 import _native

    lib = _native.load()
    fn = lib.tccl_allreduce_sum_noalloc
    fn.argtypes = [C.POINTER(C.c_uint64), C.c_int32, C.c_int32, C.c_uint64, C.c_uint64]
    fn.restype = C.c_int
    return lib, fn


def _noalloc_allreduce(fn, tensors):
    ptrs = (C.c_uint64 * len(tensors))(*[t.data_ptr() for t in tensors])
    code = DTYPES[tensors[0].dtype][0]
    return fn(ptrs, len(tensors), code, tensors[0].numel(), torch.cuda.current_stream().cuda_stream)


@pytest.mark.parametrize("dtype", list(DTYPES))
# 1001 / 1003 elements: byte counts that are no multiple of 16, so the scalar tail of both
# phases (snapshot copy and per-element sum) runs too.
@pytest.mark.parametrize("n_ranks,numel", [(2, 1000), (4, 4096), (8, 32768), (3, 72), (2, 1001),
                                           (5, 1003)])
def test_matches_heap_allreduce_two_calls_in_a_row(dtype, n_ranks, numel):
    import tileccl_b200 as tccl
    from tileccl_b200 import ops

    _, fn = _symbol()
    tol = DTYPES[dtype][1]
    torch.cuda.set_device(0)
    ctxs = tccl.init_local(n_ranks, 16 << 20, devices=[0] * n_ranks)
    try:
        gen = torch.Generator(device="cuda").manual_seed(1234 + numel)
        for call in range(2):
            data = [torch.rand(numel, device="cuda", generator=gen).mul_(2).sub_(1).to(dtype)
                    for _ in range(n_ranks)]
            # existing entry point: heap-based all-reduce on the same values
            heap_bufs = [c.zeros(numel, dtype=dtype) for c in ctxs]
            for hb, d in zip(heap_bufs, data):
                hb.copy_(d)
            for hb, c in zip(heap_bufs, ctxs):
                ops.allreduce(hb, ctx=c)
            # new entry point: ordinary device tensors, scratch inside the library
            mine = [d.clone() for d in data]
            assert _noalloc_allreduce(fn, mine) == 0
            torch.cuda.synchronize()
            for r in range(n_ranks):
                want = heap_bufs[r].float()
                err = (mine[r].float() - want).abs().max().item() / (want.abs().max().item() + 1e-9)
                assert err < tol, f"call {call}, rank {r}: rel err {err:.3e}"
            exact = sum(d.float() for d in data)
            err = (mine[0].float() - exact).abs().max().item() / (exact.abs().max().item() + 1e-9)
            assert err < tol
    finally:
        torch.cuda.synchronize()
        for c in ctxs:
            c.heap.cleanup()


def test_rejects_what_does_not_fit():
    lib, fn = _symbol()
    torch.cuda.set_device(0)
    big = [torch.zeros(256 * 1024 // 2 + 8, device="cuda", dtype=torch.float16) for _ in range(2)]
    assert _noalloc_allreduce(fn, big) != 0
    assert b"exceeds the built-in scratch" in lib.tccl_last_error()
    nine = [torch.zeros(16, device="cuda", dtype=torch.float32) for _ in range(9)]
    assert _noalloc_allreduce(fn, nine) != 0
    assert b"n_ranks" in lib.tccl_last_error()
    # an element count whose byte size wraps around 2**64 must be rejected, not run as empty
    small = [torch.zeros(16, device="cuda", dtype=torch.float16) for _ in range(2)]
    ptrs = (C.c_uint64 * 2)(*[t.data_ptr() for t in small])
    assert fn(ptrs, 2, 0, 1 << 63, torch.cuda.current_stream().cuda_stream) != 0
    assert b"exceeds the built-in scratch" in lib.tccl_last_error()
    ok = [torch.ones(256 * 1024 // 4, device="cuda", dtype=torch.float32) for _ in range(2)]
    assert _noalloc_allreduce(fn, ok) == 0            # exactly the maximum is accepted
    torch.cuda.synchronize()
    assert float(ok[0].min()) == 2.0 and float(ok[1].max()) == 2.0
