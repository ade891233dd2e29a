"""Host-side planning of the host-streamed A operand (ops/_fused.py: launch_streamed)."""
from types import SimpleNamespace as NS

import pytest

from tileccl_b200.ops._fused import _tile_row_chunks


def _plan(m_tiles, n_tiles, owners, rank, sub_m, a_rows):
    return NS(n_tiles_local=n_tiles, m_tiles_local=m_tiles, owners=owners,
              spec=NS(rank=rank, world_size=max(owners, 1), sub_m=sub_m, a_rows=a_rows,
                      split_axis=0))


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


def test_chunks_follow_owner_major_order():
    # rank 1 of 4 visits owner 2's rows first and its own rows last
    chunks = _tile_row_chunks(_plan(32, 16, 4, 1, 4096, 16384))
    assert chunks[0][2][0][0] == 2 * 4096
    assert chunks[-1][2][-1] == (1 * 4096 + 4096 - (chunks[-1][2][-1][1] - chunks[-1][2][-1][0]),
                                 2 * 4096)
