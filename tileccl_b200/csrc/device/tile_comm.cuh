// One-sided tile movement between ranks over NVLink / NVSwitch peer mappings.
// Same four verbs as the reference (tileccl/primitives/communication.py:31-225):
//   tile_remote_load / tile_remote_store  - value based (registers <-> peer memory)
//   tile_put / tile_get                   - pointer based (local memory <-> peer memory)
// plus the two NVLS forms the reference has no counterpart for:
//   tile_put_mc      - one multimem.st lands the tile in every rank's heap
//   tile_get_reduce  - multimem.ld_reduce returns the sum over all ranks
// A pointer argument named `sym_*` points into the CALLER's heap; the peer's
// copy of the object is found by translate_ptr.  In a debug build
// (-DTILECCL_DEBUG_CHECKS) a verb whose symmetric tile is not inside the caller's
// heap records the violation and moves nothing.
#pragma once
#include "tile_mem.cuh"

namespace tileccl {

template <int kMaxVec>
__device__ __forceinline__ int tile_remote_load(const SymmWindow& w, const TileView& sym_src,
                                                int from_rank, uint4 (&frag)[kMaxVec], int tid,
                                                int nthreads) {
  if (!symm_tile_ok(w, sym_src)) return 0;
  TileView s = sym_src;
  s.ptr = translate_ptr(w, sym_src.ptr, w.rank, from_rank);
  return tile_load(s, frag, tid, nthreads);
}

template <int kMaxVec>
__device__ __forceinline__ void tile_remote_store(const SymmWindow& w, const TileView& sym_dst,
                                                  int to_rank, const uint4 (&frag)[kMaxVec],
                                                  int tid, int nthreads) {
  if (!symm_tile_ok(w, sym_dst)) return;
  TileView d = sym_dst;
  d.ptr = translate_ptr(w, sym_dst.ptr, w.rank, to_rank);
  tile_store(d, frag, tid, nthreads);
}

// local `src` -> the same place as `sym_dst` in `to_rank`'s heap
__device__ __forceinline__ void tile_put(const SymmWindow& w, const TileView& src,
                                         const TileView& sym_dst, int to_rank, int tid,
                                         int nthreads) {
  if (!symm_tile_ok(w, sym_dst)) return;
  TileView d = sym_dst;
  d.ptr = translate_ptr(w, sym_dst.ptr, w.rank, to_rank);
  tile_copy<false>(d, src, tid, nthreads);
}

// `sym_src` in `from_rank`'s heap -> local `dst`
__device__ __forceinline__ void tile_get(const SymmWindow& w, const TileView& sym_src,
                                         const TileView& dst, int from_rank, int tid,
                                         int nthreads) {
  if (!symm_tile_ok(w, sym_src)) return;
  TileView s = sym_src;
  s.ptr = translate_ptr(w, sym_src.ptr, w.rank, from_rank);
  tile_copy<true>(dst, s, tid, nthreads);
}

// local `src` -> `sym_dst` in EVERY rank's heap with one store per 16 bytes.
// Requires w.mc_base != 0 and 16-byte aligned rows.
__device__ __forceinline__ void tile_put_mc(const SymmWindow& w, const TileView& src,
                                            const TileView& sym_dst, int tid, int nthreads) {
  if (!mc_span_ok(w, sym_dst.ptr, tile_span_bytes(sym_dst))) return;
  char* mc = mc_ptr(w, sym_dst.ptr);
  const int vec_per_row = src.row_bytes >> 4;
  const int total = src.rows * vec_per_row;
  for (int i = tid; i < total; i += nthreads) {
    int r = i / vec_per_row, c = i - r * vec_per_row;
    uint4 v = *reinterpret_cast<const uint4*>(src.ptr + r * src.ld_bytes + (c << 4));
    multimem_st_v4(mc + r * sym_dst.ld_bytes + (c << 4), v);
  }
}

// dst = sum over ranks of `sym_src` (16-bit floats summed with fp32 accumulation
// in the switch).  kind: 0 = fp16, 1 = bf16, 2 = fp32.
__device__ __forceinline__ void tile_get_reduce(const SymmWindow& w, const TileView& sym_src,
                                                const TileView& dst, int kind, int tid,
                                                int nthreads) {
  if (!mc_span_ok(w, sym_src.ptr, tile_span_bytes(sym_src))) return;
  const char* mc = mc_ptr(w, sym_src.ptr);
  const int vec_per_row = sym_src.row_bytes >> 4;
  const int total = sym_src.rows * vec_per_row;
  for (int i = tid; i < total; i += nthreads) {
    int r = i / vec_per_row, c = i - r * vec_per_row;
    const char* p = mc + r * sym_src.ld_bytes + (c << 4);
    uint4 v = kind == 0   ? multimem_ld_reduce_f16x8(p)
              : kind == 1 ? multimem_ld_reduce_bf16x8(p)
                          : multimem_ld_reduce_f32x4(p);
    *reinterpret_cast<uint4*>(dst.ptr + r * dst.ld_bytes + (c << 4)) = v;
  }
}

}  // namespace tileccl
