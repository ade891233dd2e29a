"""Context, symmetric heap and allocator on one GPU (single rank and emulated ranks)."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_context_single_rank():
    import tileccl_b200 as tccl

    ctx = tccl.init(backend="cuda", rank=0, world_size=1, heap_size=8 << 20, force_backend=True)
    try:
        assert ctx.has_heap and tccl.current_context() is ctx and tccl.get_world_size() == 1
        z = ctx.zeros(16, 32, dtype=torch.float16)
        r = ctx.randn((8, 8), dtype=torch.float32)
        e = ctx.empty(4, dtype=torch.bfloat16)
        assert z.shape == (16, 32) and z.device == ctx.torch_device and float(z.abs().sum()) == 0
        assert r.shape == (8, 8) and e.dtype == torch.bfloat16
        assert ctx.is_symmetric(z) and not ctx.is_symmetric(torch.zeros(4, device="cuda"))
        w1 = ctx.workspace("scratch", 64, dtype=torch.int32)
        w2 = ctx.workspace("scratch", 64, dtype=torch.int32)
        assert w1.data_ptr() == w2.data_ptr()
        assert z.data_ptr() % 256 == 0 and r.data_ptr() % 256 == 0
        s = ctx.as_symmetric(torch.arange(10, device="cuda"))
        assert ctx.is_symmetric(s) and s.tolist() == list(range(10))
        ctx.barrier()
        md = ctx.heap_metadata()
        assert md["mode"] == "local_only" and md["allocator"]["alignment"] == 256
        assert ctx.heap_bases.tolist() == [ctx.heap.local_base]
        assert ctx.support_matrix().ops["gemm_allgather"].state == "supported"
    finally:
        ctx.heap.cleanup()
        ctx.heap.cleanup()   # idempotent


def test_heap_exhaustion_and_reset():
    from tileccl_b200 import _native
    from tileccl_b200.memory import SymmetricHeap

    heap = SymmetricHeap(1 << 20, 0, 1)
    try:
        heap.allocate_tensor((1 << 19,), torch.uint8)
        with pytest.raises(_native.NativeError, match="exhausted"):
            heap.allocate_tensor((1 << 20,), torch.uint8)
        used = heap.bytes_allocated
        assert used >= 1 << 19 and heap.bytes_free == heap.size - used
        heap.reset_allocator()
        assert heap.bytes_allocated == 0
        with pytest.raises(ValueError):
            heap.get_offset(0)
    finally:
        heap.cleanup()
    with pytest.raises(RuntimeError):
        heap.allocate_tensor((4,), torch.uint8)


def test_emulated_ranks_share_one_window():
    import tileccl_b200 as tccl
    from tileccl_b200.memory import PointerTranslator

    ctxs = tccl.init_local(4, 4 << 20)
    try:
        h0 = ctxs[0].heap
        assert ctxs[0].emulated == (torch.cuda.device_count() < 4)
        assert h0.mode == "single_process" and h0.transport_strategy == "vmm_single_process"
        bases = h0.heap_bases.tolist()
        assert bases == [h0.window_base + r * h0.stride for r in range(4)]
        xs = [c.zeros(64, dtype=torch.int32) for c in ctxs]
        assert len({h0.get_offset(xs[0].data_ptr())} | {c.heap.get_offset(x.data_ptr())
                                                         for c, x in zip(ctxs, xs)}) == 1
        xs[2].fill_(7)
        assert h0.peer_view(xs[0], 2).tolist() == [7] * 64          # rank 2's copy seen from rank 0
        assert h0.translate(xs[0].data_ptr(), 2) == xs[2].data_ptr()
        tr = PointerTranslator.from_heap(h0)
        assert tr.translate(xs[0].data_ptr(), 0, 3) == xs[3].data_ptr()
        with pytest.raises(ValueError):
            tr.translate(xs[0].data_ptr(), 1, 0)                     # not inside rank 1's heap
    finally:
        torch.cuda.synchronize()
        for c in ctxs:
            c.heap.cleanup()


def test_gemm_allscatter_single_gpu_smoke():
    """Non-heap tensors are fine at world_size 1 (the reference's smoke test)."""
    import tileccl_b200 as tccl
    from tileccl_b200.memory import SymmetricHeap

    heaps = SymmetricHeap.create_all(size=64 << 20, world_size=1)
    try:
        ctx = tccl.init(backend="cuda", rank=0, world_size=1, heap=heaps[0], force_backend=True)
        a = torch.randn(128, 64, device=ctx.device, dtype=torch.float16)
        b = torch.randn(64, 128, device=ctx.device, dtype=torch.float16)
        c = torch.zeros(128, 128, device=ctx.device, dtype=torch.float16)
        tccl.ops.gemm_allscatter(a, b, c, ctx=ctx, pattern="bulk_sync")
        torch.cuda.synchronize()
        ref = torch.matmul(a.float(), b.float()).half()
        assert torch.allclose(c, ref, rtol=1e-2, atol=1e-1)
    finally:
        for h in heaps:
            h.cleanup()
