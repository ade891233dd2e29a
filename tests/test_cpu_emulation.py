"""CPU plumbing: world_size ranks emulated as threads of one process (fp32), checked
against torch, plus host-side fault injection (no GPU involved)."""

import pytest
import torch

from tileccl_b200 import emulation as em


def _inputs(ws, M, N, K, seed=0):
    g = torch.Generator().manual_seed(seed)
    return g, (lambda r, c: torch.randn(r, c, generator=g) / K ** 0.5)


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
def test_gemm_allgather_semantics(ws):
    M, N, K = 512, 256, 128
    _, rnd = _inputs(ws, M, N, K)
    A = [rnd(M // ws, K) for _ in range(ws)]
    B = [rnd(K, N) for _ in range(ws)]
    C, st = em.gemm_allgather(A, B, block_m=64, block_n=64)
    assert st.ok
    ref = torch.cat([A[r] @ B[r] for r in range(ws)])
    for c in C:
        torch.testing.assert_close(c, ref, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("ws", [1, 2, 4, 8])
def test_gemm_reducescatter_semantics(ws):
    M, N, K = 512, 256, 128
    _, rnd = _inputs(ws, M, N, K, seed=1)
    A = [rnd(M, K // ws) for _ in range(ws)]
    B = [rnd(K // ws, N) for _ in range(ws)]
    C, st = em.gemm_reducescatter(A, B, block_m=64, block_n=64, group_m_tiles=2)
    assert st.ok
    full = sum(A[r] @ B[r] for r in range(ws))
    for r in range(ws):
        torch.testing.assert_close(C[r], full[r * M // ws:(r + 1) * M // ws], rtol=1e-4, atol=1e-5)


def test_ragged_tiles():
    ws, M, N, K = 2, 200, 72, 40
    _, rnd = _inputs(ws, M, N, K, seed=2)
    A = [rnd(M // ws, K) for _ in range(ws)]
    B = [rnd(K, N) for _ in range(ws)]
    C, _ = em.gemm_allgather(A, B, block_m=64, block_n=32)
    torch.testing.assert_close(C[1], torch.cat([A[r] @ B[r] for r in range(ws)]), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("fault", ["no_signal", "short_signal", "absent"])
def test_faulty_rank_makes_peers_time_out_allgather(fault):
    ws, M, N, K = 2, 256, 128, 32
    _, rnd = _inputs(ws, M, N, K)
    A = [rnd(M // ws, K) for _ in range(ws)]
    B = [rnd(K, N) for _ in range(ws)]
    _, st = em.gemm_allgather(A, B, block_m=64, block_n=64, fault_rank=1, fault=fault,
                              timeout_ms=100, raise_on_timeout=False)
    assert st.timed_out and st.rank == 0 and st.observed < st.expected
    with pytest.raises(em.EmulatedTimeout):
        em.gemm_allgather(A, B, block_m=64, block_n=64, fault_rank=1, fault=fault, timeout_ms=50)


@pytest.mark.parametrize("fault", ["no_signal", "short_signal", "absent"])
def test_faulty_rank_makes_owner_time_out_reducescatter(fault):
    ws, M, N, K = 4, 256, 128, 64
    _, rnd = _inputs(ws, M, N, K)
    A = [rnd(M, K // ws) for _ in range(ws)]
    B = [rnd(K // ws, N) for _ in range(ws)]
    _, st = em.gemm_reducescatter(A, B, block_m=64, block_n=64, fault_rank=2, fault=fault,
                                  timeout_ms=100, raise_on_timeout=False)
    assert st.timed_out and st.rank != 2 and st.where == 40


def test_late_rank_within_budget_is_fine():
    ws, M, N, K = 2, 256, 128, 32
    _, rnd = _inputs(ws, M, N, K)
    A = [rnd(M // ws, K) for _ in range(ws)]
    B = [rnd(K, N) for _ in range(ws)]
    C, st = em.gemm_allgather(A, B, block_m=64, block_n=64, fault_rank=0, fault="late",
                              fault_delay_ms=100, timeout_ms=3000)
    assert st.ok
    _, st = em.gemm_allgather(A, B, block_m=64, block_n=64, fault_rank=0, fault="late",
                              fault_delay_ms=400, timeout_ms=50, raise_on_timeout=False)
    assert st.timed_out


def test_tile_order_own_tiles_last():
    order = em.tile_order(2, 2, owners=4, rank=1, world_size=4)
    owners = [o for o, _, _ in order]
    # rounds over the peers (rank+1, rank+2, rank+3 per tile row), own rows last
    assert owners == [2, 2, 3, 3, 0, 0] * 2 + [1] * 4
    assert [(lm, ln) for _, lm, ln in order[:6]] == [(0, 0), (0, 1)] * 3
    assert [(lm, ln) for _, lm, ln in order[-4:]] == [(0, 0), (0, 1), (1, 0), (1, 1)]
    rot = em.tile_order(4, 1, rot_m_tiles=2)
    assert [lm for _, lm, _ in rot] == [2, 3, 0, 1]


@pytest.mark.parametrize("m,n,ws,lag", [(8, 2, 2, 3), (5, 3, 4, 1), (6, 1, 8, 2), (4, 2, 3, 4),
                                         (4, 2, 3, 9)])
def test_tile_order_with_trailing_own_rows(m, n, ws, lag):
    for rank in range(ws):
        order = em.tile_order(m, n, owners=ws, rank=rank, world_size=ws, own_lag=lag)
        # a permutation of all (owner, row, column) triples
        assert sorted(order) == sorted((o, lm, ln) for o in range(ws) for lm in range(m)
                                       for ln in range(n))
        pos = {tile: i for i, tile in enumerate(order)}
        eff = lag if lag <= m else m
        for j in range(m):
            # own row j comes after every remote row j + eff - 1 (clipped to the last round) ...
            r = min(j + eff, m) - 1
            for o in range(ws):
                if o != rank:
                    assert pos[(rank, j, 0)] > pos[(o, r, n - 1)]
        # ... and at every instant all ranks address the same distance d = owner - rank
        for t in range(len(order)):
            o, lm, _ = order[t]
            o0, lm0, _ = em.tile_order(m, n, owners=ws, rank=0, world_size=ws, own_lag=lag)[t]
            assert (o - rank) % ws == o0 % ws and lm == lm0


@pytest.mark.parametrize("ws,m_tiles,lag", [(2, 6, 1), (2, 6, 3), (4, 4, 2), (8, 3, 1), (3, 5, 5),
                                            (4, 2, 7)])
def test_reducescatter_with_trailing_own_rows_is_correct_and_deadlock_free(ws, m_tiles, lag):
    """Every rank is a thread that walks the round order and blocks at its own tiles."""
    torch.manual_seed(ws * 100 + m_tiles * 10 + lag)
    bm, bn = 16, 32
    M, N, K = ws * m_tiles * bm - (3 if m_tiles > 2 else 0) * ws, 80, 8 * ws
    A = [torch.randn(M, K // ws) for _ in range(ws)]
    B = [torch.randn(K // ws, N) for _ in range(ws)]
    outs, st = em.gemm_reducescatter(A, B, block_m=bm, block_n=bn, own_lag=lag, timeout_ms=5000)
    assert st.ok
    full = sum(a @ b for a, b in zip(A, B))
    mloc = M // ws
    for r in range(ws):
        assert torch.allclose(outs[r], full[r * mloc:(r + 1) * mloc], atol=1e-4, rtol=1e-4)


def test_reducescatter_with_lag_reports_a_missing_peer():
    torch.manual_seed(3)
    A = [torch.randn(128, 8) for _ in range(2)]
    B = [torch.randn(8, 64) for _ in range(2)]
    _, st = em.gemm_reducescatter(A, B, block_m=16, block_n=32, own_lag=2, fault_rank=1,
                                  fault="absent", timeout_ms=200, raise_on_timeout=False)
    assert st.timed_out and st.rank == 0


@pytest.mark.parametrize("ws,m_tiles,lag,delay", [(2, 1, 0, 2), (4, 2, 0, 3), (4, 4, 1, 2),
                                                  (8, 2, 1, 4), (2, 6, 2, 2)])
def test_late_signalling_needs_the_flush_before_an_owner_wait(ws, m_tiles, lag, delay):
    """Signals held back while their data is in flight: with the flush before a blocking owner
    wait the schedule completes; the smallest case shows that without it the ranks stop each
    other (each holds exactly the signals its peer is waiting for)."""
    torch.manual_seed(11)
    bm, bn = 16, 32
    M, N, K = ws * m_tiles * bm, 64, 4 * ws
    A = [torch.randn(M, K // ws) for _ in range(ws)]
    B = [torch.randn(K // ws, N) for _ in range(ws)]
    outs, st = em.gemm_reducescatter(A, B, block_m=bm, block_n=bn, own_lag=lag,
                                     signal_delay_tiles=delay, timeout_ms=5000)
    assert st.ok
    full = sum(a @ b for a, b in zip(A, B))
    mloc = M // ws
    for r in range(ws):
        assert torch.allclose(outs[r], full[r * mloc:(r + 1) * mloc], atol=1e-4, rtol=1e-4)


def test_late_signalling_without_the_flush_deadlocks():
    torch.manual_seed(12)
    A = [torch.randn(32, 4) for _ in range(2)]       # one tile row of two tiles per owner
    B = [torch.randn(4, 64) for _ in range(2)]
    _, st = em.gemm_reducescatter(A, B, block_m=16, block_n=32, signal_delay_tiles=2,
                                  flush_before_wait=False, timeout_ms=300,
                                  raise_on_timeout=False)
    assert st.timed_out
