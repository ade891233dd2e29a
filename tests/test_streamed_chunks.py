"""Host-side planning of the host-streamed A operand (ops/_fused.py: launch_streamed)."""
from types import SimpleNamespace as NS

import pytest

from tileccl_b200.ops._fused import _tile_row_chunks


def _plan(m_tiles, n_tiles, owners, rank, sub_m, a_rows):
    return NS(n_tiles_local=n_tiles, m_tiles_local=m_tiles, owners=owners,
              spec=NS(rank=rank, world_size=max(owners, 1), sub_m=sub_m, a_rows=a_rows,
                      split_axis=0, rs_own_lag=0))


@pytest.mark.parametrize("m_tiles,n_tiles,owners,rank,sub_m", [
    (128, 16, 1, 0, 16384), (32, 16, 4, 1, 4096), (5, 3, 2, 0, 600), (1, 1, 1, 0, 100),
    (7, 2, 8, 5, 777)])
def test_chunks_cover_every_tile_and_row_once(m_tiles, n_tiles, owners, rank, sub_m):
    a_rows = sub_m * owners
    chunks = _tile_row_chunks(_plan(m_tiles, n_tiles, owners, rank, sub_m, a_rows), min_tiles=6)
    # tile ranges are contiguous and complete
    assert chunks[0][0] == 0 and chunks[-1][1] == m_tiles * n_tiles * owners
    for (_, e0, _), (b1, _, _) in zip(chunks, chunks[1:]):
        assert e0 == b1
    seen = [0] * a_rows
    for _, _, ranges in chunks:
        for lo, hi in ranges:
            assert 0 <= lo < hi <= a_rows
            for r in range(lo, hi):
                seen[r] += 1
    assert all(v == 1 for v in seen)


def test_chunks_follow_the_round_order():
    # rank 1 of 4: every round visits owners 2, 3, 0; its own rows come last.  The rows a
    # run needs are merged into one contiguous range per owner.
    chunks = _tile_row_chunks(_plan(32, 16, 4, 1, 4096, 16384))
    first = chunks[0][2]
    assert {lo // 4096 for lo, _ in first} == {0, 2, 3} and len(first) == 3
    assert all(lo % 4096 == 0 for lo, _ in first)            # each owner's first rows
    assert chunks[-1][2][-1][1] == 2 * 4096                  # ends with rank 1's own rows


def test_visit_rows_matches_the_native_tile_order():
    from tileccl_b200 import emulation as em
    from tileccl_b200.ops._fused import visit_rows

    for (m, ws, lag) in [(8, 2, 3), (5, 4, 1), (6, 8, 2), (4, 3, 0), (4, 3, 9)]:
        for rank in range(ws):
            native = em.tile_order(m, 2, owners=ws, rank=rank, world_size=ws, own_lag=lag)
            assert [(o, lm) for o, lm, ln in native if ln == 0] == visit_rows(m, ws, rank, ws, lag)


def test_default_rs_own_lag_policy(monkeypatch):
    from tileccl_b200.ops._fused import default_rs_own_lag

    monkeypatch.delenv("TILECCL_RS_OWN_LAG", raising=False)
    # two ranks, 64 tile rows of 16 tiles: a round is 2 MiB = ~3 us of link -> about 13 rounds
    lag = default_rs_own_lag(2, 64, 16)
    assert 8 <= lag <= 32
    # eight ranks: a round is 14.7 MiB -> a few rounds
    assert 1 <= default_rs_own_lag(8, 16, 16) <= 4
    # nothing to overlap with a single tile row, or when the lag would cover every row
    assert default_rs_own_lag(2, 1, 16) == 0
    assert default_rs_own_lag(2, 4, 1) == 0
    monkeypatch.setenv("TILECCL_RS_OWN_LAG", "5")
    assert default_rs_own_lag(2, 64, 16) == 5


def test_nvls_policy_for_collectives(monkeypatch):
    from types import SimpleNamespace
    from tileccl_b200.primitives.collectives import _use_multimem

    for var in ("TILECCL_DISABLE_NVLS", "TILECCL_FORCE_NVLS"):
        monkeypatch.delenv(var, raising=False)
    two = SimpleNamespace(has_multicast=True, world_size=2)
    eight = SimpleNamespace(has_multicast=True, world_size=8)
    none = SimpleNamespace(has_multicast=False, world_size=8)
    assert not _use_multimem(two, 1 << 20)        # a multicast store loops back at two ranks
    assert _use_multimem(eight, 1 << 20)
    assert not _use_multimem(eight, 24 + 4)       # not a multiple of 16 bytes
    assert not _use_multimem(none, 1 << 20)
    monkeypatch.setenv("TILECCL_FORCE_NVLS", "1")
    assert _use_multimem(two, 1 << 20)
    monkeypatch.setenv("TILECCL_DISABLE_NVLS", "1")
    assert not _use_multimem(eight, 1 << 20)
