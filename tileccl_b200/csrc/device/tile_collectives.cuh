// Tile collectives as device functions: all-gather, broadcast, scatter,
// reduce-scatter and all-reduce over buffers on the symmetric heap, callable
// from any kernel (the library's own collective kernel in
// kernels/collectives.cu is a thin composition of them).  Counterpart of the
// reference's tile_allreduce / tile_allgather / tile_scatter /
// tile_reduce_scatter / tile_broadcast (tileccl/primitives/collectives.py:484-831).
//
// Two layers:
//
//   data movement   tile_allgather, tile_broadcast, tile_scatter,
//                   tile_reduce_scatter, tile_allreduce_chunk.  No waiting inside:
//                   like the reference's device functions they assume that the
//                   buffers they touch are ready, and the caller orders them.
//                   NVSwitch gives every pair of GPUs full bandwidth, so every
//                   algorithm is direct (one hop): push for all-gather / broadcast /
//                   scatter, pull-and-sum for reduce-scatter, pull-sum-push for
//                   all-reduce.  With `use_mc` (an NVLS mapping is bound and sizes
//                   are 16-byte multiples) one multimem.st reaches every rank and
//                   one multimem.ld_reduce returns the sum over all ranks.
//
//   protocol        tile_coll_announce / tile_coll_wait_ready / tile_coll_publish /
//                   tile_coll_wait_done: the three-phase handshake on a symmetric
//                   counter block whose counters only grow (epoch = 1, 2, 3 ... per
//                   call), every wait bounded.  tile_allreduce etc. with a
//                   TileCollSync argument run the whole call: announce, wait, move,
//                   publish, wait.
//
// Cooperation: every function takes a TileCoop {tid, nthreads}: the calling
// thread's index among the threads that share the work.  That may be a warp, a
// CTA (`tile_coop_cta()`) or the whole grid (`tile_coop_grid()`).  The protocol
// functions are CTA-collective (they use __syncthreads) and must be called by all
// threads of the CTA.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "tile_comm.cuh"
#include "tile_compute.cuh"
#include "tile_sync.cuh"

namespace tileccl {

static constexpr int kTileCollMaxRanks = 8;
// Counter block layout (uint32, on the symmetric heap, zero before first use):
//   [0, 8)   ready[src]   phase-1 announcements received from rank src
//   [8, 16)  done[src]    phase-2 completions received from rank src
//   [16]     cta_done     local: CTAs of the current call that finished phase 2
static constexpr int kTileCollCounters = 32;

enum TileDtype : int { kTileF16 = 0, kTileBF16 = 1, kTileF32 = 2, kTileBytes = 3 };

struct TileCoop {
  uint64_t tid;       // this thread's index among the cooperating threads
  uint64_t nthreads;  // how many threads cooperate
};
__device__ __forceinline__ TileCoop tile_coop_cta() {
  return TileCoop{threadIdx.x, blockDim.x};
}
__device__ __forceinline__ TileCoop tile_coop_grid() {
  return TileCoop{static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x,
                  static_cast<uint64_t>(gridDim.x) * blockDim.x};
}
__device__ __forceinline__ TileCoop tile_coop_warp() {
  return TileCoop{threadIdx.x & 31u, 32u};
}

// ---------------------------------------------------------------------------
// building blocks
// ---------------------------------------------------------------------------
namespace coll_detail {

template <typename T>
__device__ __forceinline__ T* peer_of(const SymmWindow& w, T* local, int r) {
  return translate_ptr(w, local, w.rank, r);
}

__device__ __forceinline__ bool vec16_ok(const void* a, const void* b, uint64_t bytes) {
  return ((reinterpret_cast<uint64_t>(a) | reinterpret_cast<uint64_t>(b) | bytes) & 15u) == 0;
}

template <typename T>
__device__ __forceinline__ void copy_elems(char* dst, const char* src, uint64_t bytes,
                                           const TileCoop& c) {
  const uint64_t n = bytes / sizeof(T);
  for (uint64_t i = c.tid; i < n; i += c.nthreads)
    reinterpret_cast<T*>(dst)[i] = reinterpret_cast<const T*>(src)[i];
}

// Copy from local memory to one (possibly remote) destination: 16 bytes per access
// with kU loads in flight per thread when alignment allows, else one element per
// access (chunk offsets of odd-sized messages are only element-aligned).
template <int kU = 8>
__device__ __forceinline__ void copy_vec(char* dst, const char* src, uint64_t bytes, int elem_size,
                                         const TileCoop& c) {
  if (vec16_ok(dst, src, bytes)) {
    const uint64_t n = bytes >> 4;
    uint64_t i = c.tid;
    for (; i + (kU - 1) * c.nthreads < n; i += kU * c.nthreads) {
      uint4 v[kU];
#pragma unroll
      for (int j = 0; j < kU; ++j)
        v[j] = *reinterpret_cast<const uint4*>(src + ((i + j * c.nthreads) << 4));
#pragma unroll
      for (int j = 0; j < kU; ++j) st_remote_v4(dst + ((i + j * c.nthreads) << 4), v[j]);
    }
    for (; i < n; i += c.nthreads)
      st_remote_v4(dst + (i << 4), *reinterpret_cast<const uint4*>(src + (i << 4)));
  } else if (elem_size == 8) {
    copy_elems<uint64_t>(dst, src, bytes, c);
  } else if (elem_size == 4) {
    copy_elems<uint32_t>(dst, src, bytes, c);
  } else if (elem_size == 2) {
    copy_elems<uint16_t>(dst, src, bytes, c);
  } else {
    copy_elems<uint8_t>(dst, src, bytes, c);
  }
}

// Copy from local memory to the multicast alias: one store lands in every rank's heap.
template <int kU = 8>
__device__ __forceinline__ void copy_vec_mc(char* mc_dst, const char* src, uint64_t bytes,
                                            const TileCoop& c) {
  const uint64_t n = bytes >> 4;
  uint64_t i = c.tid;
  for (; i + (kU - 1) * c.nthreads < n; i += kU * c.nthreads) {
    uint4 v[kU];
#pragma unroll
    for (int j = 0; j < kU; ++j)
      v[j] = *reinterpret_cast<const uint4*>(src + ((i + j * c.nthreads) << 4));
#pragma unroll
    for (int j = 0; j < kU; ++j) multimem_st_v4(mc_dst + ((i + j * c.nthreads) << 4), v[j]);
  }
  for (; i < n; i += c.nthreads)
    multimem_st_v4(mc_dst + (i << 4), *reinterpret_cast<const uint4*>(src + (i << 4)));
}

__device__ __forceinline__ float4 as_f4(const uint4& v) {
  return make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z),
                     __uint_as_float(v.w));
}
// acc (8 floats for 16-bit types, 4 for fp32) += v
__device__ __forceinline__ void accumulate(int dtype, float* acc, const uint4& v) {
  if (dtype == kTileF32) {
    float4 f = as_f4(v);
    acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
  } else {
    tile_accumulate_16x8(dtype == kTileBF16, acc, v);
  }
}
__device__ __forceinline__ uint4 finish(int dtype, const float* acc) {
  if (dtype == kTileF32)
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]),
                      __float_as_uint(acc[3]));
  return tile_cast_f32x8(dtype == kTileBF16, acc);
}
__device__ __forceinline__ uint4 mc_reduce(int dtype, const void* mc) {
  return dtype == kTileF32 ? multimem_ld_reduce_f32x4(mc)
                           : dtype == kTileBF16 ? multimem_ld_reduce_bf16x8(mc)
                                                : multimem_ld_reduce_f16x8(mc);
}
__device__ __forceinline__ float load_scalar(int dtype, const char* q) {
  return dtype == kTileF32 ? *reinterpret_cast<const volatile float*>(q)
         : dtype == kTileBF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(q))
                              : __half2float(*reinterpret_cast<const __half*>(q));
}
__device__ __forceinline__ void store_scalar(int dtype, char* q, float a) {
  if (dtype == kTileF32) *reinterpret_cast<float*>(q) = a;
  else if (dtype == kTileBF16) *reinterpret_cast<__nv_bfloat16*>(q) = __float2bfloat16(a);
  else *reinterpret_cast<__half*>(q) = __float2half(a);
}

// Sum `my_bytes` at byte offset `chunk_off` of `sym_src` over all ranks (fp32
// accumulation, rank order) and write the result either to the local `dst_local`
// (reduce-scatter) or back to offset `chunk_off` of `sym_dst` in EVERY rank's heap
// (the second half of an all-reduce).
template <bool kToAll>
__device__ __forceinline__ void reduce_chunk(const SymmWindow& w, const char* sym_src,
                                             char* dst_local, char* sym_dst, uint64_t chunk_off,
                                             uint64_t my_bytes, int dtype, bool use_mc,
                                             const TileCoop& c) {
  const int ws = w.world_size;
  // Offsets of a chunk are only element-aligned when the chunk is not a multiple of
  // 16 bytes: then everything goes through the scalar loop at the end.
  const bool aligned =
      ((chunk_off | reinterpret_cast<uint64_t>(kToAll ? sym_dst : dst_local) |
        reinterpret_cast<uint64_t>(sym_src)) & 15u) == 0;
  const uint64_t n = aligned ? (my_bytes >> 4) : 0;
  uint64_t i = c.tid;
  if (use_mc) {
    // In-switch reduction: kU multimem.ld_reduce in flight per thread, then the stores
    // (one multimem.st reaches every rank).
    constexpr int kU = 8;
    const char* mc_src = mc_ptr(w, const_cast<char*>(sym_src)) + chunk_off;
    char* mc_dst = kToAll ? mc_ptr(w, sym_dst) + chunk_off : nullptr;
    for (; i + (kU - 1) * c.nthreads < n; i += kU * c.nthreads) {
      uint4 o[kU];
#pragma unroll
      for (int j = 0; j < kU; ++j) o[j] = mc_reduce(dtype, mc_src + ((i + j * c.nthreads) << 4));
#pragma unroll
      for (int j = 0; j < kU; ++j) {
        const uint64_t ii = i + j * c.nthreads;
        if (kToAll) multimem_st_v4(mc_dst + (ii << 4), o[j]);
        else *reinterpret_cast<uint4*>(dst_local + (ii << 4)) = o[j];
      }
    }
    for (; i < n; i += c.nthreads) {
      const uint4 o = mc_reduce(dtype, mc_src + (i << 4));
      if (kToAll) multimem_st_v4(mc_dst + (i << 4), o);
      else *reinterpret_cast<uint4*>(dst_local + (i << 4)) = o;
    }
  } else {
    // Peer loads of two items in flight per thread before the first accumulate.
    for (; i + c.nthreads < n; i += 2 * c.nthreads) {
      uint4 v0[kTileCollMaxRanks], v1[kTileCollMaxRanks];
      const uint64_t off0 = chunk_off + (i << 4), off1 = chunk_off + ((i + c.nthreads) << 4);
#pragma unroll
      for (int r = 0; r < kTileCollMaxRanks; ++r)
        if (r < ws) {
          v0[r] = ld_remote_v4(peer_of(w, sym_src, r) + off0);
          v1[r] = ld_remote_v4(peer_of(w, sym_src, r) + off1);
        }
      float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int r = 0; r < kTileCollMaxRanks; ++r)
        if (r < ws) {
          accumulate(dtype, a0, v0[r]);
          accumulate(dtype, a1, v1[r]);
        }
      const uint4 o0 = finish(dtype, a0), o1 = finish(dtype, a1);
      if (!kToAll) {
        *reinterpret_cast<uint4*>(dst_local + (i << 4)) = o0;
        *reinterpret_cast<uint4*>(dst_local + ((i + c.nthreads) << 4)) = o1;
      } else {
#pragma unroll
        for (int r = 0; r < kTileCollMaxRanks; ++r)
          if (r < ws) {
            st_remote_v4(peer_of(w, sym_dst, r) + off0, o0);
            st_remote_v4(peer_of(w, sym_dst, r) + off1, o1);
          }
      }
    }
    for (; i < n; i += c.nthreads) {
      const uint64_t off = chunk_off + (i << 4);
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 v[kTileCollMaxRanks];
#pragma unroll
      for (int r = 0; r < kTileCollMaxRanks; ++r)
        if (r < ws) v[r] = ld_remote_v4(peer_of(w, sym_src, r) + off);
#pragma unroll
      for (int r = 0; r < kTileCollMaxRanks; ++r)
        if (r < ws) accumulate(dtype, acc, v[r]);
      const uint4 out = finish(dtype, acc);
      if (!kToAll) {
        *reinterpret_cast<uint4*>(dst_local + (i << 4)) = out;
      } else {
#pragma unroll
        for (int r = 0; r < kTileCollMaxRanks; ++r)
          if (r < ws) st_remote_v4(peer_of(w, sym_dst, r) + off, out);
      }
    }
  }
  // scalar remainder: the < 16-byte tail, or the whole chunk when it is unaligned
  if ((n << 4) < my_bytes) {
    const int es = dtype == kTileF32 ? 4 : 2;
    for (uint64_t b = (n << 4) + c.tid * es; b < my_bytes; b += c.nthreads * es) {
      float a = 0.f;
      for (int r = 0; r < ws; ++r) a += load_scalar(dtype, peer_of(w, sym_src, r) + chunk_off + b);
      if (!kToAll) {
        store_scalar(dtype, dst_local + b, a);
      } else {
        for (int r = 0; r < ws; ++r) store_scalar(dtype, peer_of(w, sym_dst, r) + chunk_off + b, a);
      }
    }
  }
}

}  // namespace coll_detail

// ---------------------------------------------------------------------------
// data movement (no waiting inside)
// ---------------------------------------------------------------------------

// Slot `rank` of `sym_dst` in every rank's heap <- this rank's `bytes` at `src`
// (`src` is any local memory; `sym_dst` holds world_size * bytes).
__device__ __forceinline__ void tile_allgather(const SymmWindow& w, const void* src, void* sym_dst,
                                               uint64_t bytes, int elem_size, bool use_mc,
                                               const TileCoop& c) {
  const char* s = static_cast<const char*>(src);
  char* d = static_cast<char*>(sym_dst);
  if (!symm_span_ok(w, d, bytes * w.world_size, w.rank)) return;   // debug build only
  if (use_mc && (bytes & 15u) == 0) {
    coll_detail::copy_vec_mc(mc_ptr(w, d) + w.rank * bytes, s, bytes, c);
  } else {
    for (int k = 0; k < w.world_size; ++k) {
      const int r = (w.rank + k) % w.world_size;   // start with this rank, peers staggered
      coll_detail::copy_vec(coll_detail::peer_of(w, d, r) + w.rank * bytes, s, bytes, elem_size, c);
    }
  }
}

// Root's `bytes` at `sym_buf` -> the same place in every other rank's heap.
__device__ __forceinline__ void tile_broadcast(const SymmWindow& w, void* sym_buf, uint64_t bytes,
                                               int root, int elem_size, bool use_mc,
                                               const TileCoop& c) {
  if (w.rank != root) return;
  char* b = static_cast<char*>(sym_buf);
  if (!symm_span_ok(w, b, bytes, w.rank)) return;                  // debug build only
  if (use_mc && (bytes & 15u) == 0) {
    coll_detail::copy_vec_mc(mc_ptr(w, b), b, bytes, c);
  } else {
    for (int k = 1; k < w.world_size; ++k)
      coll_detail::copy_vec(coll_detail::peer_of(w, b, (w.rank + k) % w.world_size), b, bytes,
                            elem_size, c);
  }
}

// Root's chunk r (`bytes` each, at `src`) -> `sym_dst` of rank r.
__device__ __forceinline__ void tile_scatter(const SymmWindow& w, const void* src, void* sym_dst,
                                             uint64_t bytes, int root, int elem_size,
                                             const TileCoop& c) {
  if (w.rank != root) return;
  const char* s = static_cast<const char*>(src);
  char* d = static_cast<char*>(sym_dst);
  if (!symm_span_ok(w, d, bytes, w.rank)) return;                  // debug build only
  for (int k = 0; k < w.world_size; ++k) {
    const int r = (w.rank + k) % w.world_size;
    coll_detail::copy_vec(coll_detail::peer_of(w, d, r), s + r * bytes, bytes, elem_size, c);
  }
}

// `dst` (local, `bytes`) <- sum over ranks of chunk `rank` of `sym_src` (world_size * bytes).
__device__ __forceinline__ void tile_reduce_scatter(const SymmWindow& w, const void* sym_src,
                                                    void* dst, uint64_t bytes, int dtype,
                                                    bool use_mc, const TileCoop& c) {
  if (!symm_span_ok(w, static_cast<const char*>(sym_src), bytes * w.world_size, w.rank)) return;
  coll_detail::reduce_chunk<false>(w, static_cast<const char*>(sym_src), static_cast<char*>(dst),
                                   nullptr, w.rank * bytes, bytes, dtype, use_mc, c);
}

// The data phase of a two-shot all-reduce on `sym_buf` (`bytes` in every heap): this
// rank sums its 1 / world_size share over all ranks and writes the sums back into
// every rank's buffer.  Shares are 16-byte multiples; the last may be short or empty.
__device__ __forceinline__ void tile_allreduce_chunk(const SymmWindow& w, void* sym_buf,
                                                     uint64_t bytes, int dtype, bool use_mc,
                                                     const TileCoop& c) {
  const uint64_t ws = static_cast<uint64_t>(w.world_size);
  const uint64_t chunk = ((bytes + ws - 1) / ws + 15) & ~static_cast<uint64_t>(15);
  const uint64_t off = w.rank * chunk;
  const uint64_t mine = off >= bytes ? 0 : (bytes - off < chunk ? bytes - off : chunk);
  char* b = static_cast<char*>(sym_buf);
  if (!symm_span_ok(w, b, bytes, w.rank)) return;                  // debug build only
  coll_detail::reduce_chunk<true>(w, b, nullptr, b, off, mine, dtype, use_mc, c);
}

// ---------------------------------------------------------------------------
// protocol (CTA-collective; every wait bounded)
// ---------------------------------------------------------------------------
struct TileCollSync {
  uint32_t* counters;   // this rank's counter block (kTileCollCounters words, symmetric)
  uint32_t epoch;       // 1, 2, 3 ... per call on this block
  uint32_t* status;     // optional status words (ptx.cuh), may be null
  int root;             // rooted ops (broadcast / scatter): the root; else -1
};

namespace coll_detail {
// counter[offset + rank] += 1 in the heap of every rank of the dependency set
// (thread r of the CTA signals rank r).
__device__ __forceinline__ void signal_set(const SymmWindow& w, const TileCollSync& s, int offset,
                                           int only_rank) {
  uint32_t* ctr = s.counters + offset + w.rank;
  const int r = threadIdx.x;
  if (r < w.world_size && r != w.rank && (only_rank < 0 || r == only_rank))
    red_release_sys_add(peer_of(w, ctr, r), 1u);
}
// Wait until counter[offset + r] >= epoch for every r of the dependency set (thread r polls).
__device__ __forceinline__ bool wait_set(const SymmWindow& w, const TileCollSync& s, int offset,
                                         int only_rank, const WaitBudget& wb, uint32_t where) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  const int r = threadIdx.x;
  if (r < w.world_size && r != w.rank && (only_rank < 0 || r == only_rank)) {
    uint32_t seen = 0;
    if (!tile_wait_ge(s.counters + offset + r, s.epoch, wb, &seen)) {
      report_status(s.status, kStatusTimeoutSignal, where, s.epoch, seen, w.rank, r);
      failed = 1;
    }
  }
  __syncthreads();
  return failed == 0;
}
}  // namespace coll_detail

// Phase 1, one CTA per rank: "my buffers for this call are ready / may be overwritten".
// A rooted op only needs receivers -> root; the others need all -> all.
__device__ __forceinline__ void tile_coll_announce(const SymmWindow& w, const TileCollSync& s) {
  if (s.root < 0) coll_detail::signal_set(w, s, 0, -1);
  else if (w.rank != s.root) coll_detail::signal_set(w, s, 0, s.root);
}
// Phase 2 entry, every CTA that moves data: wait for the announcements it depends on.
__device__ __forceinline__ bool tile_coll_wait_ready(const SymmWindow& w, const TileCollSync& s,
                                                     const WaitBudget& wb) {
  if (s.root < 0) return coll_detail::wait_set(w, s, 0, -1, wb, 60);
  if (w.rank == s.root) return coll_detail::wait_set(w, s, 0, -1, wb, 61);
  return true;
}
// Phase 2 exit, every CTA that moved data (`n_ctas` of them): the last one to get here
// tells the ranks that depend on this rank's data that it is complete.
__device__ __forceinline__ void tile_coll_publish(const SymmWindow& w, const TileCollSync& s,
                                                  uint32_t n_ctas) {
  __shared__ int is_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t* cta_done = s.counters + 16;
    const uint32_t old = atomicAdd(cta_done, 1u);
    is_last = (old == n_ctas - 1) ? 1 : 0;
    if (is_last) *cta_done = 0;
  }
  __syncthreads();
  if (is_last) {
    __threadfence_system();
    if (s.root < 0 || w.rank == s.root) coll_detail::signal_set(w, s, 8, -1);
  }
}
// Phase 3, one CTA per rank: wait for the completions this rank depends on.
__device__ __forceinline__ bool tile_coll_wait_done(const SymmWindow& w, const TileCollSync& s,
                                                    const WaitBudget& wb) {
  if (s.root < 0) return coll_detail::wait_set(w, s, 8, -1, wb, 62);
  if (w.rank != s.root) return coll_detail::wait_set(w, s, 8, s.root, wb, 63);
  return true;
}

// ---------------------------------------------------------------------------
// pipelined relay broadcast (large messages, three or more ranks)
// ---------------------------------------------------------------------------
// A multimem.st broadcast is bounded by what ONE source can multicast, and a root that
// unicasts to n - 1 peers sends every byte n - 1 times.  Here the root sends every byte
// ONCE: the buffer is cut into pieces, piece p goes to relay rank relay_rank_of(p) (the
// non-root ranks in turn) together with a flag, and that rank forwards the piece to the
// other non-root ranks as soon as the flag shows the current call.  Root egress is B,
// every other rank receives B and sends (n - 2) / (n - 1) B: all links run at the unicast
// rate and the transfer is pipelined piece by piece.
//
// `flags` is a symmetric uint32[kTileRelayMaxPieces] that only ever holds call numbers
// (epoch = 1, 2, 3 ... per call on this flag block; zero before first use).  Both functions
// are CTA-collective; CTA `cta` of `n_ctas` takes every n_ctas-th piece.  `bytes` and
// `piece_bytes` are multiples of 16.
static constexpr uint32_t kTileRelayMaxPieces = 16384;

__device__ __forceinline__ int relay_rank_of(uint32_t piece, int root, int world_size) {
  const int k = static_cast<int>(piece % static_cast<uint32_t>(world_size - 1));
  return k < root ? k : k + 1;                       // k-th rank that is not the root
}

namespace coll_detail {
// 16-byte copy of `n` vectors by one CTA with up to kU loads in flight per thread for ANY
// n (the slots past the end are predicated off): pieces are a few vectors per thread, and
// without the loads up front every store would wait for its own load.
template <int kU>
__device__ __forceinline__ void copy_piece(char* dst, const char* src, uint64_t n) {
  for (uint64_t base = threadIdx.x; base < n; base += static_cast<uint64_t>(kU) * blockDim.x) {
    uint4 v[kU];
#pragma unroll
    for (int j = 0; j < kU; ++j) {
      const uint64_t i = base + static_cast<uint64_t>(j) * blockDim.x;
      if (i < n) v[j] = ld_remote_v4(src + (i << 4));
    }
#pragma unroll
    for (int j = 0; j < kU; ++j) {
      const uint64_t i = base + static_cast<uint64_t>(j) * blockDim.x;
      if (i < n) st_remote_v4(dst + (i << 4), v[j]);
    }
  }
}
}  // namespace coll_detail

// Root: piece p -> the same place in relay_rank_of(p)'s heap, then flag[p] = epoch there.
__device__ __forceinline__ void tile_relay_push(const SymmWindow& w, void* sym_buf, uint64_t bytes,
                                                uint64_t piece_bytes, uint32_t* sym_flags,
                                                uint32_t epoch, uint32_t cta, uint32_t n_ctas) {
  char* b = static_cast<char*>(sym_buf);
  if (!symm_span_ok(w, b, bytes, w.rank)) return;                  // debug build only
  const uint32_t n_pieces = static_cast<uint32_t>((bytes + piece_bytes - 1) / piece_bytes);
  for (uint32_t p = cta; p < n_pieces; p += n_ctas) {
    const uint64_t off = static_cast<uint64_t>(p) * piece_bytes;
    const uint64_t len = bytes - off < piece_bytes ? bytes - off : piece_bytes;
    const int to = relay_rank_of(p, w.rank, w.world_size);
    coll_detail::copy_piece<8>(coll_detail::peer_of(w, b, to) + off, b + off, len >> 4);
    __syncthreads();                                 // every thread's stores are issued ...
    if (threadIdx.x == 0) {
      __threadfence_system();                        // ... and ordered before the flag
      st_release_sys(coll_detail::peer_of(w, sym_flags, to) + p, epoch);
    }
  }
}

// Relay (every rank but the root): wait for each of its pieces, copy it from the local
// buffer to the other non-root ranks.  Returns false when a piece never arrived within the
// budget (the status words then name the piece).
__device__ __forceinline__ bool tile_relay_forward(const SymmWindow& w, void* sym_buf,
                                                   uint64_t bytes, uint64_t piece_bytes, int root,
                                                   const uint32_t* sym_flags, uint32_t epoch,
                                                   uint32_t cta, uint32_t n_ctas,
                                                   const WaitBudget& wb, uint32_t* status) {
  __shared__ int arrived;
  char* b = static_cast<char*>(sym_buf);
  if (!symm_span_ok(w, b, bytes, w.rank)) return true;             // debug build only
  const int ws = w.world_size;
  const uint32_t n_pieces = static_cast<uint32_t>((bytes + piece_bytes - 1) / piece_bytes);
  const uint32_t mine = static_cast<uint32_t>(w.rank < root ? w.rank : w.rank - 1);
  // destination k = 1 .. ws - 1 is rank (rank + k) % ws (peers staggered), the root left out
  auto dest = [&](int k) -> char* {
    const int r = (w.rank + k) % ws;
    return r == root ? nullptr : coll_detail::peer_of(w, b, r);
  };
  for (uint32_t p = cta * static_cast<uint32_t>(ws - 1) + mine; p < n_pieces;
       p += n_ctas * static_cast<uint32_t>(ws - 1)) {
    if (threadIdx.x == 0) {
      uint32_t seen = 0;
      arrived = tile_wait_ge(sym_flags + p, epoch, wb, &seen) ? 1 : 0;
      if (!arrived) report_status(status, kStatusTimeoutSignal, 65, epoch, seen, w.rank, p);
    }
    __syncthreads();
    if (!arrived) return false;
    const uint64_t off = static_cast<uint64_t>(p) * piece_bytes;
    const uint64_t n = (bytes - off < piece_bytes ? bytes - off : piece_bytes) >> 4;
    constexpr int kU = 4;                            // loads in flight per thread, any n
    for (uint64_t base = threadIdx.x; base < n; base += static_cast<uint64_t>(kU) * blockDim.x) {
      uint4 v[kU];
#pragma unroll
      for (int j = 0; j < kU; ++j) {
        const uint64_t i = base + static_cast<uint64_t>(j) * blockDim.x;
        if (i < n) v[j] = ld_remote_v4(b + off + (i << 4));
      }
      for (int k = 1; k < ws; ++k) {
        char* d = dest(k);
        if (d == nullptr) continue;
#pragma unroll
        for (int j = 0; j < kU; ++j) {
          const uint64_t i = base + static_cast<uint64_t>(j) * blockDim.x;
          if (i < n) st_remote_v4(d + off + (i << 4), v[j]);
        }
      }
    }
    __syncthreads();                                 // `arrived` is rewritten for the next piece
  }
  return true;
}

// ---------------------------------------------------------------------------
// whole calls from inside a user kernel: ONE CTA per rank runs announce -> wait ->
// move -> publish -> wait.  Every rank must make the same call with the same epoch.
// Returns false when a wait ran out of its budget (the status words then say where).
// ---------------------------------------------------------------------------
__device__ __forceinline__ bool tile_allreduce(const SymmWindow& w, void* sym_buf, uint64_t bytes,
                                               int dtype, bool use_mc, const TileCollSync& s,
                                               const WaitBudget& wb) {
  tile_coll_announce(w, s);
  bool ok = tile_coll_wait_ready(w, s, wb);
  if (ok) tile_allreduce_chunk(w, sym_buf, bytes, dtype, use_mc, tile_coop_cta());
  tile_coll_publish(w, s, 1);
  return tile_coll_wait_done(w, s, wb) && ok;
}
__device__ __forceinline__ bool tile_allgather(const SymmWindow& w, const void* src, void* sym_dst,
                                               uint64_t bytes, int elem_size, bool use_mc,
                                               const TileCollSync& s, const WaitBudget& wb) {
  tile_coll_announce(w, s);
  bool ok = tile_coll_wait_ready(w, s, wb);
  if (ok) tile_allgather(w, src, sym_dst, bytes, elem_size, use_mc, tile_coop_cta());
  tile_coll_publish(w, s, 1);
  return tile_coll_wait_done(w, s, wb) && ok;
}
__device__ __forceinline__ bool tile_reduce_scatter(const SymmWindow& w, const void* sym_src,
                                                    void* dst, uint64_t bytes, int dtype,
                                                    bool use_mc, const TileCollSync& s,
                                                    const WaitBudget& wb) {
  tile_coll_announce(w, s);
  bool ok = tile_coll_wait_ready(w, s, wb);
  if (ok) tile_reduce_scatter(w, sym_src, dst, bytes, dtype, use_mc, tile_coop_cta());
  tile_coll_publish(w, s, 1);
  return tile_coll_wait_done(w, s, wb) && ok;
}
__device__ __forceinline__ bool tile_broadcast(const SymmWindow& w, void* sym_buf, uint64_t bytes,
                                               int elem_size, bool use_mc, const TileCollSync& s,
                                               const WaitBudget& wb) {
  tile_coll_announce(w, s);
  bool ok = tile_coll_wait_ready(w, s, wb);
  if (ok) tile_broadcast(w, sym_buf, bytes, s.root, elem_size, use_mc, tile_coop_cta());
  tile_coll_publish(w, s, 1);
  return tile_coll_wait_done(w, s, wb) && ok;
}
__device__ __forceinline__ bool tile_scatter(const SymmWindow& w, const void* src, void* sym_dst,
                                             uint64_t bytes, int elem_size, const TileCollSync& s,
                                             const WaitBudget& wb) {
  tile_coll_announce(w, s);
  bool ok = tile_coll_wait_ready(w, s, wb);
  if (ok) tile_scatter(w, src, sym_dst, bytes, s.root, elem_size, tile_coop_cta());
  tile_coll_publish(w, s, 1);
  return tile_coll_wait_done(w, s, wb) && ok;
}

}  // namespace tileccl
