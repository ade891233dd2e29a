"""A operand streamed from pinned host memory by the op itself (``a_host=``)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(got, ref):
    return (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-9)


@pytest.fixture()
def ctx():
    import tileccl_b200 as tccl

    c = tccl.init(heap_size=1 << 30)
    yield c
    torch.cuda.synchronize()
    c.heap.cleanup()


@pytest.mark.parametrize("shape", [(8192, 4096, 512), (1000, 768, 320), (128, 256, 64)])
def test_allgather_rows_from_host(ctx, shape):
    from tileccl_b200 import ops

    M, N, K = shape
    a_host = (torch.randn(M, K) * K ** -0.5).to(torch.float16).pin_memory()
    a = ctx.zeros(M, K, dtype=torch.float16)
    b = ctx.randn(K, N, dtype=torch.float16)
    c = ctx.zeros(M, N, dtype=torch.float16)
    for it in range(2):                      # second call: the copy must wait for the first launch
        if it:
            a_host.mul_(-1.0)
        ops.gemm_allgather_rows(a, b, c, ctx=ctx, a_host=a_host)
        torch.cuda.synchronize()
        ref = a_host.cuda().float() @ b.float()
        assert torch.equal(a.cpu(), a_host)
        assert _rel(c, ref) < 5e-3


def test_reducescatter_rows_from_host(ctx):
    from tileccl_b200 import ops

    M, N, K = 4096, 2048, 1024
    a_host = (torch.randn(M, K) * K ** -0.5).to(torch.bfloat16).pin_memory()
    a = ctx.zeros(M, K, dtype=torch.bfloat16)
    b = ctx.randn(K, N, dtype=torch.bfloat16)
    c = ctx.zeros(M, N, dtype=torch.bfloat16)
    ops.gemm_reducescatter_rows(a, b, c, ctx=ctx, a_host=a_host)
    torch.cuda.synchronize()
    assert _rel(c, a_host.cuda().float() @ b.float()) < 2e-2


def test_rejects_pageable_or_mismatched_host_tensor(ctx):
    from tileccl_b200 import ops

    a = ctx.zeros(256, 64, dtype=torch.float16)
    b = ctx.randn(64, 256, dtype=torch.float16)
    c = ctx.zeros(256, 256, dtype=torch.float16)
    with pytest.raises(ValueError):
        ops.gemm_allgather_rows(a, b, c, ctx=ctx, a_host=torch.zeros(256, 64, dtype=torch.float16))
    with pytest.raises(ValueError):
        ops.gemm_allgather_rows(a, b, c, ctx=ctx,
                                a_host=torch.zeros(128, 64, dtype=torch.float16).pin_memory())


def test_plan_ordered_copies_pipeline_two_problems(ctx):
    """``a_host_order="plan"``: the copy of one problem may overlap the kernels of the other;
    repeated calls on the same buffers still see each call's own data."""
    from tileccl_b200 import ops

    probs = []
    for (M, N, K) in ((4096, 2048, 512), (2048, 4096, 1024)):
        a_host = (torch.randn(M, K) * K ** -0.5).to(torch.float16).pin_memory()
        probs.append((a_host, ctx.zeros(M, K, dtype=torch.float16),
                      ctx.randn(K, N, dtype=torch.float16), ctx.zeros(M, N, dtype=torch.float16)))
    for it in range(3):
        for a_host, a, b, c in probs:
            a_host.mul_(-0.5)
        for a_host, a, b, c in probs:
            ops.gemm_allgather_rows(a, b, c, ctx=ctx, a_host=a_host, a_host_order="plan")
        torch.cuda.synchronize()
        for a_host, a, b, c in probs:
            assert torch.equal(a.cpu(), a_host)
            assert _rel(c, a_host.cuda().float() @ b.float()) < 5e-3
