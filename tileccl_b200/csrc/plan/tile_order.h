// The order in which a rank visits output tiles, shared by the sm_100a kernel
// (kernels/gemm_sm100.cu) and the CPU emulator (cpu_emul/fake_device.cc) so that
// both execute the same schedule.
//
// With `owners` > 1 (reduce-scatter) a rank works in rounds: round r produces tile
// row r of the sub-problem of rank+1, then of rank+2, ... rank+owners-1 (at any
// moment all ranks send to "their rank + d" for the same d, a permutation, so no
// receiver is oversubscribed), and every owner gets row r of all its partial sums
// after round r.  The rank's own (reducing) rows follow `own_lag` rounds behind:
// own row j is visited at the end of round j + own_lag, when the peers' partials
// for it have long arrived, so the reduction overlaps the link-bound rounds; the
// last own_lag own rows run after the final round.  own_lag = 0 keeps all own
// rows for the end (remote tiles first, then own tiles, each range contiguous).
// Inside a tile row the column tiles run left to right; TileGroups, which are
// bands of tile rows of one owner, therefore complete in order.
#pragma once

#if defined(__CUDACC__)
#define TCCL_HD __host__ __device__ __forceinline__
#else
#define TCCL_HD inline
#endif

namespace tileccl {

struct TileOrderShape {
  int m_tiles_local, n_tiles_local;  // tiles of one owner's sub-problem
  int owners;                        // 1, or world_size
  int rank, world_size;
  int rot_m_tiles;                   // owners == 1: first tile row to visit (wraps around)
  int own_lag;                       // owners > 1: rounds by which own rows trail (0 = all last)
};

struct TileOrderEntry {
  int owner;   // rank that owns the tile (== rank when owners == 1)
  int lm, ln;  // tile row / column inside the owner's sub-problem
};

TCCL_HD int tile_order_count(const TileOrderShape& s) {
  return s.m_tiles_local * s.n_tiles_local * s.owners;
}

TCCL_HD TileOrderEntry tile_order_decode(const TileOrderShape& s, int t) {
  TileOrderEntry e;
  const int row = t / s.n_tiles_local;      // tile row in visiting order
  e.ln = t - row * s.n_tiles_local;
  if (s.owners <= 1) {
    e.lm = row;
    if (s.rot_m_tiles != 0) {
      e.lm += s.rot_m_tiles;
      if (e.lm >= s.m_tiles_local) e.lm -= s.m_tiles_local;
    }
    e.owner = s.rank;
    return e;
  }
  const int m = s.m_tiles_local, w = s.owners;
  const int lag = (s.own_lag <= 0 || s.own_lag > m) ? m : s.own_lag;
  const int head = lag * (w - 1);           // rounds [0, lag): remote rows only
  const int mid = (m - lag) * w;            // rounds [lag, m): remote rows + one own row
  int d;                                    // distance to the owner, 0 = this rank
  if (row < head) {
    e.lm = row / (w - 1);
    d = row - e.lm * (w - 1) + 1;
  } else if (row < head + mid) {
    const int r2 = row - head;
    const int round = lag + r2 / w;
    const int k = r2 - (r2 / w) * w;
    if (k < w - 1) { e.lm = round; d = k + 1; }
    else { e.lm = round - lag; d = 0; }
  } else {
    e.lm = (m - lag) + (row - head - mid);
    d = 0;
  }
  e.owner = (s.rank + d) % s.world_size;
  return e;
}

}  // namespace tileccl
