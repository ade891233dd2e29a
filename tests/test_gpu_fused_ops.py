"""Fused GEMM + collective operators with several ranks driven by one process.

With fewer GPUs than ranks the ranks are emulated on shared GPUs (launches are
replayed phase by phase, no kernel waits on another one), so these tests run on a
single B200 and exercise the same kernels, addressing and signalling as a
multi-GPU run."""

import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = {torch.float16: 5e-3, torch.bfloat16: 2e-2}


def _rel(got, ref):
    return (got.float() - ref.float()).abs().max().item() / (ref.float().abs().max().item() + 1e-9)


@pytest.fixture(params=[2, 4, 8])
def ctxs(request):
    import tileccl_b200 as tccl

    cs = tccl.init_local(request.param, 512 << 20)
    yield cs
    for d in range(torch.cuda.device_count()):
        torch.cuda.synchronize(d)
    for c in cs:
        c.heap.cleanup()


def _randn(ctx, r, c, dtype, scale=1.0):
    t = ctx.randn(r, c, dtype=dtype)
    if scale != 1.0:
        t.mul_(scale)
    return t


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_allgather_rows(ctxs, dtype):
    from tileccl_b200 import ops

    ws = len(ctxs)
    M, N, K = 256 * ws, 768, 320
    A = [_randn(c, M // ws, K, dtype, K ** -0.5) for c in ctxs]
    B = [_randn(c, K, N, dtype) for c in ctxs]
    C = [c.zeros(M, N, dtype=dtype) for c in ctxs]
    for _ in range(3):                                   # epochs advance, counters are not reset
        for r, c in enumerate(ctxs):
            ops.gemm_allgather_rows(A[r], B[r], C[r], ctx=c)
    for c in ctxs:
        ops.check_status(c)
    ref = torch.cat([A[r].float().cpu() @ B[r].float().cpu() for r in range(ws)])
    for r in range(ws):
        assert _rel(C[r].cpu(), ref) < TOL[dtype]


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_gemm_reducescatter_rows(ctxs, dtype):
    from tileccl_b200 import ops

    ws = len(ctxs)
    M, N, K = 128 * ws * 2, 512, 64 * ws
    A = [_randn(c, M, K // ws, dtype, K ** -0.5) for c in ctxs]
    B = [_randn(c, K // ws, N, dtype) for c in ctxs]
    C = [torch.zeros(M // ws, N, dtype=dtype, device=c.torch_device) for c in ctxs]
    for _ in range(4):                                   # staging parity alternates per call
        for r, c in enumerate(ctxs):
            ops.gemm_reducescatter_rows(A[r], B[r], C[r], ctx=c)
    for c in ctxs:
        ops.check_status(c)
    full = sum(A[r].float().cpu() @ B[r].float().cpu() for r in range(ws))
    for r in range(ws):
        assert _rel(C[r].cpu(), full[r * M // ws:(r + 1) * M // ws]) < TOL[dtype]


def test_reference_column_contracts(ctxs):
    from tileccl_b200 import ops

    ws, dtype = len(ctxs), torch.float16
    M, N, K = 384, 256 * ws, 128
    A = [_randn(c, M, K, dtype, K ** -0.5) for c in ctxs]
    Bs = [_randn(c, K, N // ws, dtype) for c in ctxs]
    C = [c.zeros(M, N, dtype=dtype) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.gemm_allgather(A[r], Bs[r], C[r], ctx=c)
    ref = torch.cat([A[r].float().cpu() @ Bs[r].float().cpu() for r in range(ws)], dim=1)
    for r in range(ws):
        assert _rel(C[r].cpu(), ref) < TOL[dtype]
    Bf = [_randn(c, K, N, dtype) for c in ctxs]
    Cs = [c.zeros(M, N // ws, dtype=dtype) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.gemm_reducescatter(A[r], Bf[r], Cs[r], ctx=c)
    full = sum(A[r].float().cpu() @ Bf[r].float().cpu() for r in range(ws))
    for r in range(ws):
        assert _rel(Cs[r].cpu(), full[:, r * N // ws:(r + 1) * N // ws]) < TOL[dtype]
    for c in ctxs:
        ops.check_status(c)


@pytest.mark.parametrize("pattern", ["bulk_sync", "fused_sequential", "producer_consumer",
                                     "wg_specialized", "auto", "fused_seq", "pc", "wg_spec"])
def test_gemm_allscatter_patterns(ctxs, pattern):
    from tileccl_b200 import ops

    ws, dtype = len(ctxs), torch.float16
    M, N, K = 512, 64 * ws * 2, 192
    torch.manual_seed(3)
    a = (torch.randn(M, K) / K ** 0.5).to(dtype)
    b = torch.randn(K, N).to(dtype)
    A = [a.to(c.torch_device) for c in ctxs]
    B = [b.to(c.torch_device) for c in ctxs]
    C = [c.zeros(M, N, dtype=dtype) for c in ctxs]
    for _ in range(2):
        for r, c in enumerate(ctxs):
            ops.gemm_allscatter(A[r], B[r], C[r], ctx=c, pattern=pattern)
    for c in ctxs:
        ops.check_status(c)
    ref = a.float() @ b.float()
    for r in range(ws):
        assert _rel(C[r].cpu(), ref) < TOL[dtype]


def test_allscatter_own_slice_is_never_overwritten(ctxs):
    """full/full all-scatter with a different A per rank: peers only ever write the slices they
    own, so a rank's own column slice must hold its own product.  (The other slices are
    written both locally and by their owners, which is only well defined when every rank
    multiplies the same operands - the contract of this operator.)"""
    from tileccl_b200 import ops

    ws, dtype = len(ctxs), torch.float16
    M, N, K = 256, 64 * ws, 64
    A = [_randn(c, M, K, dtype, K ** -0.5) for c in ctxs]
    torch.manual_seed(5)
    b = torch.randn(K, N).to(dtype)
    B = [b.to(c.torch_device) for c in ctxs]
    C = [c.zeros(M, N, dtype=dtype) for c in ctxs]
    for r, c in enumerate(ctxs):
        ops.gemm_allscatter(A[r], B[r], C[r], ctx=c, pattern="fused_sequential")
    for c in ctxs:
        ops.check_status(c)
    n = N // ws
    for r in range(ws):
        want = (A[r].float().cpu() @ b.float())[:, r * n:(r + 1) * n]
        assert _rel(C[r].cpu()[:, r * n:(r + 1) * n], want) < TOL[dtype]


def test_mixed_layout_and_sharded(ctxs):
    from tileccl_b200 import ops

    ws, dtype = len(ctxs), torch.bfloat16
    M, N, K = 256, 64 * ws, 128
    c0 = ctxs[0]
    a = _randn(c0, M, K, dtype, K ** -0.5)
    b = _randn(c0, K, N, dtype)
    cs = c0.zeros(M, N // ws, dtype=dtype)
    plan = ops.build_gemm_allscatter_plan(a, b, cs, ctx=c0, b_layout="full", c_layout="shard")
    assert type(plan).__name__ == "GemmAllScatterMixedLayoutPlan" and plan.to_dict()["op"] == "gemm_allscatter"
    plan.execute(a, b, cs)
    torch.cuda.synchronize()
    assert _rel(cs.cpu(), (a.float() @ b.float())[:, :N // ws].cpu()) < TOL[dtype]
    with pytest.raises(ValueError):
        ops.gemm_allscatter(a, b[:, :N // ws].contiguous(), c0.zeros(M, N, dtype=dtype), ctx=c0,
                            b_layout="shard", c_layout="full", full_N=N)


def test_contract_errors(ctxs):
    from tileccl_b200 import ops

    c = ctxs[0]
    ws = len(ctxs)
    a = c.zeros(128, 64, dtype=torch.float16)
    b = c.zeros(64, 128, dtype=torch.float16)
    with pytest.raises(ValueError):     # output not on the heap
        ops.gemm_allgather_rows(a, b, torch.zeros(128 * ws, 128, device=c.torch_device, dtype=torch.float16), ctx=c)
    with pytest.raises(ValueError):     # wrong output shape
        ops.gemm_allgather_rows(a, b, c.zeros(128, 128, dtype=torch.float16), ctx=c) if ws > 1 else (_ for _ in ()).throw(ValueError())
    with pytest.raises(ValueError):     # dtype mismatch
        ops.gemm_reducescatter(a, b.bfloat16(), c.zeros(128, 128 // ws, dtype=torch.float16), ctx=c)
    with pytest.raises(ValueError):
        ops.gemm_reducescatter(a, b, c.zeros(128, 128 // ws, dtype=torch.float16), ctx=c, implementation="reference")
    with pytest.raises(ValueError):
        ops.gemm_allscatter(a, b, c.zeros(128, 128, dtype=torch.float16), ctx=c, pattern="telepathy")


def test_fused_kernel_abort_path_then_normal_call(ctxs, monkeypatch):
    """The owner phase of a reduce-scatter launched with no producer before it: the producer
    warp's wait for the peers' TileGroups runs out (site 40), every role of the kernel winds
    down (loads drained, MMAs committed, TMEM freed) and the launch returns.  The same
    context then runs a normal call."""
    from tileccl_b200 import ops
    from tileccl_b200.kernels.fused_gemm import TileCCLTimeoutError
    from tileccl_b200.ops import _fused

    ws, dtype = len(ctxs), torch.float16
    if not ctxs[0].emulated:
        pytest.skip("phase-split launches exist for ranks that share a GPU")
    monkeypatch.setenv("TILECCL_WAIT_BUDGET_US", "3000")     # baked into the plans built below
    M, N, K = 128 * ws * 2, 512, 64 * ws
    A = [_randn(c, M, K // ws, dtype, K ** -0.5) for c in ctxs]
    B = [_randn(c, K // ws, N, dtype) for c in ctxs]
    C = [torch.zeros(M // ws, N, dtype=dtype, device=c.torch_device) for c in ctxs]

    def run_all():
        for r, c in enumerate(ctxs):
            ops.gemm_reducescatter_rows(A[r], B[r], C[r], ctx=c)
        for c in ctxs:
            ops.check_status(c)

    run_all()
    c0 = ctxs[0]
    plans = [st["plan"] for key, st in c0._state["ops"].items()
             if isinstance(key, tuple) and key[0] == "reduce_scatter" and "plan" in st]
    assert len(plans) == 1
    plan = plans[0]
    n_remote = plan.tiles_per_owner * (ws - 1)
    with torch.cuda.device(c0.torch_device):
        plan.launch(epoch=2, tile_begin=n_remote)            # epoch 2 was never produced
    with pytest.raises(TileCCLTimeoutError) as err:
        ops.check_status(c0)
    assert "'where': 40" in str(err.value) and "peer signal" in str(err.value)
    run_all()                                                # status cleared, counters untouched
    full = sum(A[r].float().cpu() @ B[r].float().cpu() for r in range(ws))
    for r in range(ws):
        assert _rel(C[r].cpu(), full[r * M // ws:(r + 1) * M // ws]) < TOL[dtype]
    # recover(): counters and epochs restart from zero, collectively, and calls keep working
    for c in ctxs:
        ops.recover(c)
    run_all()
    for r in range(ws):
        assert _rel(C[r].cpu(), full[r * M // ws:(r + 1) * M // ws]) < TOL[dtype]


def test_call_stats_count_bytes_signals_and_tiles(ctxs):
    """Per-call counters of the fused kernel: bytes stored into peers, signals, tiles."""
    from tileccl_b200 import ops

    ws, dtype = len(ctxs), torch.float16
    M, N, K = 256 * ws, 512, 128
    A = [_randn(c, M // ws, K, dtype, K ** -0.5) for c in ctxs]
    B = [_randn(c, K, N, dtype) for c in ctxs]
    C = [c.zeros(M, N, dtype=dtype) for c in ctxs]
    for c in ctxs:
        ops.call_stats(c)                                  # clear
    for r, c in enumerate(ctxs):
        ops.gemm_allgather_rows(A[r], B[r], C[r], ctx=c)
    for c in ctxs:
        ops.check_status(c)
    for c in ctxs:
        st = ops.call_stats(c)
        assert st["bytes_pushed"] == (ws - 1) * (M // ws) * N * 2
        assert st["tiles"] == 2 * (N // 256)               # 256 rows per rank = 2 tile rows
        assert st["signals_sent"] == (ws - 1) * st["tiles"] * 4   # one per 32-row slab and peer
        assert ops.call_stats(c)["bytes_pushed"] == 0      # reading resets
