// The order in which a rank visits output tiles, shared by the sm_100a kernel
// (kernels/gemm_sm100.cu) and the CPU emulator (cpu_emul/fake_device.cc) so that
// both execute the same schedule.
//
// A rank's tile list is owner-major: with `owners` > 1 (reduce-scatter) it first
// produces the tiles owned by rank+1, then rank+2, ... and its own tiles last, so
// that remote owners receive their partial sums as early as possible and the
// local reduction finds them already there.  Inside one owner's sub-problem tiles
// run row band by row band (all column tiles of a tile row, then the next row):
// TileGroups, which are bands of tile rows, therefore complete in order.
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
  const int per_owner = s.m_tiles_local * s.n_tiles_local;
  int oi = 0, rem = t;
  if (s.owners > 1) {
    oi = t / per_owner;
    rem = t - oi * per_owner;
  }
  e.lm = rem / s.n_tiles_local;
  e.ln = rem - e.lm * s.n_tiles_local;
  if (s.owners == 1 && s.rot_m_tiles != 0) {
    e.lm += s.rot_m_tiles;
    if (e.lm >= s.m_tiles_local) e.lm -= s.m_tiles_local;
  }
  e.owner = s.owners > 1 ? (s.rank + 1 + oi) % s.world_size : s.rank;
  return e;
}

}  // namespace tileccl
