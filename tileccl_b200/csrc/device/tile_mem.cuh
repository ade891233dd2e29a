// CTA/warp-cooperative movement of a BMxBN tile of a row-major matrix, 16 bytes
// per access, with predicated tails.  Counterpart of the reference's
// tile_load / tile_store / tile_copy (tileccl/primitives/memory.py:14-165);
// here a "tile" is described by pointer + leading dimension instead of a block
// of Triton offsets.
#pragma once
#include "symm_ptr.cuh"

namespace tileccl {

// View of a tile inside a row-major matrix of `elem_bytes`-sized elements.
struct TileView {
  char* ptr;          // address of element (0, 0) of the tile
  int64_t ld_bytes;   // bytes between consecutive rows
  int rows;           // valid rows (tail tiles have fewer than BM)
  int row_bytes;      // valid bytes per row (tail tiles have fewer than BN * elem)
};

__host__ __device__ __forceinline__ TileView make_tile_view(void* base, int64_t ld_elems,
                                                            int elem_bytes, int row0, int col0,
                                                            int bm, int bn, int total_rows,
                                                            int total_cols) {
  TileView t;
  t.ptr = static_cast<char*>(base) + (static_cast<int64_t>(row0) * ld_elems + col0) * elem_bytes;
  t.ld_bytes = ld_elems * elem_bytes;
  int r = total_rows - row0;
  int c = total_cols - col0;
  t.rows = r < bm ? (r < 0 ? 0 : r) : bm;
  t.row_bytes = (c < bn ? (c < 0 ? 0 : c) : bn) * elem_bytes;
  return t;
}

// Bytes from the first to one past the last byte of the tile.
__host__ __device__ __forceinline__ uint64_t tile_span_bytes(const TileView& t) {
  if (t.rows <= 0 || t.row_bytes <= 0) return 0;
  return static_cast<uint64_t>(t.rows - 1) * static_cast<uint64_t>(t.ld_bytes) +
         static_cast<uint64_t>(t.row_bytes);
}
// Debug-build guard (see symm_ptr.cuh): the tile lies inside the CALLER's heap.
__host__ __device__ __forceinline__ bool symm_tile_ok(const SymmWindow& w, const TileView& t) {
  return symm_span_ok(w, t.ptr, tile_span_bytes(t), w.rank);
}

// Copies `src` to `dst` with `nthreads` cooperating threads (thread id `tid`).
// Rows whose start and length are 16-byte aligned move as uint4; the rest byte-wise.
template <bool kRemoteSrc = false>
__device__ __forceinline__ void tile_copy(const TileView& dst, const TileView& src, int tid,
                                          int nthreads) {
  const int rows = src.rows < dst.rows ? src.rows : dst.rows;
  const int row_bytes = src.row_bytes < dst.row_bytes ? src.row_bytes : dst.row_bytes;
  const bool vec_ok = ((reinterpret_cast<uint64_t>(src.ptr) | reinterpret_cast<uint64_t>(dst.ptr) |
                        static_cast<uint64_t>(src.ld_bytes) | static_cast<uint64_t>(dst.ld_bytes) |
                        static_cast<uint64_t>(row_bytes)) & 15u) == 0;
  if (vec_ok) {
    const int vec_per_row = row_bytes >> 4;
    const int total = rows * vec_per_row;
    for (int i = tid; i < total; i += nthreads) {
      int r = i / vec_per_row, c = i - r * vec_per_row;
      const char* s = src.ptr + r * src.ld_bytes + (c << 4);
      char* d = dst.ptr + r * dst.ld_bytes + (c << 4);
      uint4 v = kRemoteSrc ? ld_remote_v4(s) : *reinterpret_cast<const uint4*>(s);
      st_remote_v4(d, v);
    }
  } else {
    const int total = rows * row_bytes;
    for (int i = tid; i < total; i += nthreads) {
      int r = i / row_bytes, c = i - r * row_bytes;
      dst.ptr[r * dst.ld_bytes + c] = src.ptr[r * src.ld_bytes + c];
    }
  }
}

// tile_load / tile_store into / from a per-thread register fragment of uint4:
// thread `tid` owns vectors tid, tid + nthreads, ... of the tile (row-major).
template <int kMaxVec>
__device__ __forceinline__ int tile_load(const TileView& src, uint4 (&frag)[kMaxVec], int tid,
                                         int nthreads) {
  const int vec_per_row = src.row_bytes >> 4;
  const int total = src.rows * vec_per_row;
  int n = 0;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    int i = tid + k * nthreads;
    if (i < total) {
      int r = i / vec_per_row, c = i - r * vec_per_row;
      frag[k] = ld_remote_v4(src.ptr + r * src.ld_bytes + (c << 4));
      n = k + 1;
    }
  }
  return n;
}
template <int kMaxVec>
__device__ __forceinline__ void tile_store(const TileView& dst, const uint4 (&frag)[kMaxVec],
                                           int tid, int nthreads) {
  const int vec_per_row = dst.row_bytes >> 4;
  const int total = dst.rows * vec_per_row;
#pragma unroll
  for (int k = 0; k < kMaxVec; ++k) {
    int i = tid + k * nthreads;
    if (i < total) {
      int r = i / vec_per_row, c = i - r * vec_per_row;
      st_remote_v4(dst.ptr + r * dst.ld_bytes + (c << 4), frag[k]);
    }
  }
}

}  // namespace tileccl
