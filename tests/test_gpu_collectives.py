"""Tile collectives and device primitives on ranks driven by one process."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _rel(got, ref):
    return (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-9)


@pytest.fixture(params=[2, 4, 8])
def ctxs(request):
    import tileccl_b200 as tccl

    cs = tccl.init_local(request.param, 256 << 20)
    yield cs
    for d in range(torch.cuda.device_count()):
        torch.cuda.synchronize(d)
    for c in cs:
        c.heap.cleanup()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
@pytest.mark.parametrize("numel", [1024, 8198, 300_000, 2_000_000])
def test_all_five_collectives(ctxs, dtype, numel):
    from tileccl_b200 import ops
    from tileccl_b200.primitives import collectives as coll

    ws = len(ctxs)
    n = numel // ws * ws
    tol = 2e-2 if dtype is not torch.float32 else 1e-5
    xs = [c.randn(n, dtype=dtype) for c in ctxs]
    orig = [x.clone() for x in xs]
    total = sum(o.float().cpu() for o in orig)
    for rep in range(2):                                  # second call reuses counters / staging
        for r, c in enumerate(ctxs):
            xs[r].copy_(orig[r])
        for r, c in enumerate(ctxs):
            ops.allreduce(xs[r], ctx=c)
        for r in range(ws):
            assert _rel(xs[r].cpu(), total) < tol
    outs = [c.zeros(n * ws, dtype=dtype) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.allgather(orig[r], outs[r], ctx=c) if c.is_symmetric(orig[r]) else ops.allgather(xs[r].copy_(orig[r]), outs[r], ctx=c)
    cat = torch.cat([o.cpu() for o in orig])
    for r in range(ws):
        assert torch.equal(outs[r].cpu(), cat)
    src = [c.randn(n, dtype=dtype) for c in ctxs]
    part = [c.zeros(n // ws, dtype=dtype) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.reduce_scatter(src[r], part[r], ctx=c)
    tot = sum(s.float().cpu() for s in src)
    for r in range(ws):
        assert _rel(part[r].cpu(), tot[r * (n // ws):(r + 1) * (n // ws)]) < tol
    root = ws - 1
    want = src[root].cpu().clone()
    for r, c in enumerate(ctxs):
        ops.broadcast(src[r], ctx=c, root=root)
    for r in range(ws):
        assert torch.equal(src[r].cpu(), want)
    sc = [c.zeros(n // ws, dtype=dtype) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.scatter(xs[r], sc[r], ctx=c, root=0)
    root_data = xs[0].cpu()
    for r in range(ws):
        assert torch.equal(sc[r].cpu(), root_data[r * (n // ws):(r + 1) * (n // ws)])
    for c in ctxs:
        coll.check_status(c.heap)


def test_rooted_collectives_with_alternating_roots(ctxs):
    """broadcast / scatter accept any root on any call (every root has its own counters)."""
    from tileccl_b200 import ops
    from tileccl_b200.primitives import collectives as coll

    ws = len(ctxs)
    n = 4096 * ws
    bufs = [c.zeros(n, dtype=torch.float32) for c in ctxs]
    outs = [c.zeros(n // ws, dtype=torch.float32) for c in ctxs]
    for call, root in enumerate([0, 1, 0, ws - 1, 1, 0]):
        for r in range(ws):
            bufs[r].fill_(float(100 * call + r))
        for r, c in enumerate(ctxs):
            ops.broadcast(bufs[r], ctx=c, root=root)
        for r in range(ws):
            assert float(bufs[r].min()) == float(bufs[r].max()) == float(100 * call + root), (call, r)
        for r in range(ws):
            bufs[r].copy_(torch.arange(n, device=bufs[r].device, dtype=torch.float32) + 1000 * r)
        for r, c in enumerate(ctxs):
            ops.scatter(bufs[r], outs[r], ctx=c, root=root)
        for r in range(ws):
            want = torch.arange(r * (n // ws), (r + 1) * (n // ws), dtype=torch.float32) + 1000 * root
            assert torch.equal(outs[r].cpu(), want), (call, r)
    for c in ctxs:
        coll.check_status(c.heap)


@pytest.mark.parametrize("bulk", ["1", "0"])
@pytest.mark.parametrize("nbytes, threshold", [(2 << 20, 65536), ((12 << 20) + 4096 * 16, 8 << 20)])
def test_relay_broadcast_large_messages(ctxs, nbytes, threshold, bulk, monkeypatch):
    """Three or more ranks, large message: the root sends every piece once and the other
    ranks forward theirs.  Roots alternate and sizes repeat, so flags and counters of
    several calls are exercised; a guard region after the buffer must stay untouched."""
    from tileccl_b200 import ops
    from tileccl_b200.primitives import collectives as coll

    ws = len(ctxs)
    if ws < 3:
        pytest.skip("the relay needs three ranks")
    if threshold is not None:
        monkeypatch.setenv("TILECCL_BCAST_RELAY_MIN_BYTES", str(threshold))
    monkeypatch.setenv("TILECCL_BCAST_RELAY_BULK", bulk)     # bulk copies / register copies
    n = nbytes // 4
    bufs = [c.zeros(n, dtype=torch.float32) for c in ctxs]
    guards = [c.zeros(4096, dtype=torch.int32) for c in ctxs]
    for g in guards:
        g.fill_(0x5A5A5A5A)
    assert coll._relay_ok(ctxs[0].heap, nbytes, bufs[0].data_ptr())
    for call, root in enumerate([0, ws - 1, 1, 0]):
        want = None
        for r in range(ws):
            gen = torch.Generator(device=bufs[r].device).manual_seed(100 * call + r)
            bufs[r].copy_(torch.rand(n, device=bufs[r].device, generator=gen))
            if r == root:
                want = bufs[r].cpu().clone()
        for r, c in enumerate(ctxs):
            ops.broadcast(bufs[r], ctx=c, root=root)
        for r in range(ws):
            assert torch.equal(bufs[r].cpu(), want), (call, root, r)
    for c in ctxs:
        coll.check_status(c.heap)
    assert ("coll_relay", "broadcast_relay:0") in ctxs[0].heap._state
    for g in guards:
        assert int((g != 0x5A5A5A5A).sum()) == 0


def test_reset_allocator_drops_internal_workspaces(ctxs):
    """reset -> allocate -> all-reduce and fused op: library counters and staging are re-created
    instead of aliasing the tensors allocated after the reset."""
    from tileccl_b200 import ops

    ws = len(ctxs)
    xs = [c.randn(4096, dtype=torch.float32) for c in ctxs]
    for x, c in zip(xs, ctxs):
        ops.allreduce(x, ctx=c)                       # creates counters + one-shot staging
    M, N, K = 256 * ws, 256, 128
    A = [c.randn(M // ws, K, dtype=torch.float16) for c in ctxs]
    B = [c.randn(K, N, dtype=torch.float16) for c in ctxs]
    Cs = [c.zeros(M, N, dtype=torch.float16) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.gemm_allgather_rows(A[r], B[r], Cs[r], ctx=c)
    for c in ctxs:
        ops.check_status(c)
    for c in ctxs:
        c.barrier()
    for c in ctxs:
        c.heap.reset_allocator()
    assert all(c.heap.bytes_allocated == 0 for c in ctxs)
    # new user tensors now sit where the old counters / staging were; fill them with a pattern
    guard = [c.empty(1 << 16, dtype=torch.int32) for c in ctxs]
    for g in guard:
        g.fill_(0x5A5A5A5A)
    ys = [c.randn(4096, dtype=torch.float32) for c in ctxs]
    want = sum(y.float().cpu() for y in ys)
    for y, c in zip(ys, ctxs):
        ops.allreduce(y, ctx=c)
    for y in ys:
        assert _rel(y.cpu(), want) < 1e-5
    A = [c.randn(M // ws, K, dtype=torch.float16) for c in ctxs]
    B = [c.randn(K, N, dtype=torch.float16) for c in ctxs]
    Cs = [c.zeros(M, N, dtype=torch.float16) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.gemm_allgather_rows(A[r], B[r], Cs[r], ctx=c)
    for c in ctxs:
        ops.check_status(c)
    ref = torch.cat([A[r].float().cpu() @ B[r].float().cpu() for r in range(ws)])
    for r in range(ws):
        assert _rel(Cs[r].cpu(), ref) < 2e-2
    for g in guard:
        assert int((g != 0x5A5A5A5A).sum()) == 0     # nothing of the library's wrote into user memory


def test_allreduce_plan_metadata(ctxs):
    from tileccl_b200 import ops

    c = ctxs[0]
    small = ops.build_allreduce_plan(c.zeros(1024, dtype=torch.float16), ctx=c)
    big = ops.build_allreduce_plan(c.zeros(1 << 20, dtype=torch.float16), ctx=c)
    odd = ops.build_allreduce_plan(c.zeros(1001, dtype=torch.float16), ctx=c)
    assert small.implementation == "device_one_shot_ll" and small.message_regime == "latency"
    assert odd.implementation == "device_one_shot"       # not a multiple of 8 bytes: staged copy
    assert big.implementation == "device_two_shot" and big.message_regime == "bandwidth"
    assert big.to_dict()["num_chunks"] == len(ctxs)
    with pytest.raises(ValueError):
        ops.build_allreduce_plan(c.zeros(8, dtype=torch.float16), ctx=c, op="max")
    with pytest.raises(ValueError):
        ops.allgather(torch.zeros(8, device=c.torch_device), c.zeros(8 * len(ctxs), dtype=torch.float32), ctx=c)


def test_primitives_put_get_signal_wait_atomics(ctxs):
    from tileccl_b200.primitives import harness

    h0, h1 = ctxs[0].heap, ctxs[1].heap
    a0 = h0.allocate_tensor((1024,), torch.int32)
    a1 = h1.allocate_tensor((1024,), torch.int32)
    f0 = h0.allocate_signal_buffer(8)
    f1 = h1.allocate_signal_buffer(8)
    a0.copy_(torch.arange(1024, dtype=torch.int32))
    a1.zero_()
    assert harness.translate(h0, a0.data_ptr(), 1) == a1.data_ptr()
    harness.run(h0, "put", peer=1, a=a0.data_ptr(), b=a0.data_ptr(), nbytes=4096)
    assert torch.equal(a1.cpu(), a0.cpu())
    a1.mul_(2)
    harness.run(h0, "get", peer=1, a=a0.data_ptr(), b=a0.data_ptr(), nbytes=4096)
    assert torch.equal(a0.cpu(), a1.cpu())
    a0.add_(1)
    harness.run(h0, "remote_store", peer=1, a=a0.data_ptr(), b=a0.data_ptr(), nbytes=4096)
    assert torch.equal(a1.cpu(), a0.cpu())
    a1.add_(5)
    harness.run(h0, "remote_load", peer=1, a=a0.data_ptr(), b=a0.data_ptr(), nbytes=4096)
    assert torch.equal(a0.cpu(), a1.cpu())
    # flags: signal on the peer, consuming wait, bounded time-out afterwards
    harness.run(h0, "signal", peer=1, a=f0.data_ptr())
    assert f1[0].item() == 1
    assert harness.run(h1, "poll", a=f1.data_ptr())[0] == 1 and f1[0].item() == 1
    assert harness.run(h1, "wait", a=f1.data_ptr())[0] == 1 and f1[0].item() == 0
    assert harness.run(h1, "wait", a=f1.data_ptr(), budget_us=2000)[0] == 0      # nothing sets it
    assert harness.run(h1, "try_wait", a=f1.data_ptr(), value=64)[0] == 0
    # counters
    harness.run(h0, "signal_add", peer=1, a=f0.data_ptr() + 4, value=3)
    assert harness.run(h1, "wait_ge", a=f1.data_ptr() + 4, value=3)[:1] == [1]
    assert harness.run(h1, "wait_ge", a=f1.data_ptr() + 4, value=5, budget_us=2000)[:2] == [0, 3]
    # remote atomics on counter word 1 (currently 3)
    for name, val, expect in (("add", 5, 8), ("max", 100, 100), ("min", 7, 7), ("or", 8, 15),
                              ("and", 12, 12), ("xor", 5, 9), ("xchg", 42, 42)):
        harness.atomic(h0, name, f0.data_ptr() + 4, val, 1)
        assert f1[1].item() == expect, name
    assert harness.atomic(h0, "cas", f0.data_ptr() + 4, 42, 1, value2=77) == 42 and f1[1].item() == 77
    assert harness.atomic(h0, "cas", f0.data_ptr() + 4, 1, 1, value2=5) == 77 and f1[1].item() == 77
    # credits: a pool of 2 on rank 1, a third acquire times out, a remote release refills it
    f1[2] = 2
    assert harness.run(h1, "credit", a=f1.data_ptr() + 8, sub_op=0)[0] == 1
    assert harness.run(h1, "credit", a=f1.data_ptr() + 8, sub_op=0)[0] == 1
    assert harness.run(h1, "credit", a=f1.data_ptr() + 8, sub_op=0, budget_us=2000)[0] == 0
    harness.run(h0, "credit", peer=1, a=f0.data_ptr() + 8, sub_op=1)
    assert harness.run(h1, "credit", a=f1.data_ptr() + 8, sub_op=0)[0] == 1


def test_device_timeout_is_reported_and_gpu_stays_usable(ctxs):
    """A wait that nothing satisfies returns an error status; the context keeps working."""
    from tileccl_b200.kernels.fused_gemm import TileCCLTimeoutError
    from tileccl_b200.ops import _fused

    c = ctxs[0]
    sig = c.workspace("never_signalled", len(ctxs) * _fused.MAX_GROUPS, dtype=torch.int32)
    per_epoch = torch.ones(1, dtype=torch.int32, device=c.torch_device)
    import os
    os.environ["TILECCL_WAIT_BUDGET_US"] = "3000"
    try:
        with torch.cuda.device(c.torch_device):
            _fused.wait_groups(c, sig, 1, per_epoch, 1)
        with pytest.raises(TileCCLTimeoutError, match="peer signal"):
            _fused.check_status(c)
    finally:
        del os.environ["TILECCL_WAIT_BUDGET_US"]
    x = torch.ones(16, device=c.torch_device)
    assert float((x * 2).sum()) == 32.0
    _fused.check_status(c)          # status was cleared
