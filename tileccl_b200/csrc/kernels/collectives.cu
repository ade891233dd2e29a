// Tile collectives on symmetric-heap buffers: all-gather, reduce-scatter,
// all-reduce, broadcast, scatter.  One multi-CTA kernel per call; data moves with
// 16-byte peer loads/stores over NVLink, or with multimem.st / multimem.ld_reduce
// through the NVSwitch when an NVLS mapping is bound.
//
// NVSwitch gives every pair of GPUs full bandwidth, so every algorithm is direct
// (one hop): push for all-gather / broadcast / scatter, pull for reduce-scatter,
// pull-reduce + push for all-reduce (one-shot through a staging copy for small
// messages).  The reference's device collectives are ring or staged-slot kernels
// with at most 16 CTAs and 16 KiB chunks (tileccl/primitives/collectives.py:484-1615).
//
// Every call runs the same three-phase protocol on counters that only grow
// (`epoch` = 1, 2, 3 ... per call on a counter block):
//   phase 1  announce: "my buffers for this call are ready / may be overwritten"
//   phase 2  wait for the announcements it depends on, move data, publish "done"
//   phase 3  wait for the peers' "done" it depends on
// A launch normally runs all three (phase_mask = 7).  When several ranks are
// emulated on ONE GPU their kernels must not wait on one another, so the host
// issues the phases as separate launches, each for all ranks in turn.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include "../api.h"
#include "../device/ptx.cuh"
#include "../device/tile_collectives.cuh"
#include "../device/tile_ll.cuh"
#include "../runtime/errors.h"

namespace tileccl {

enum CollOp : int {
  kAllGather = 0,
  kReduceScatter = 1,
  kAllReduceTwoShot = 2,
  kAllReduceOneShot = 3,
  kBroadcast = 4,
  kScatter = 5,
};
enum CollDtype : int { kF16 = kTileF16, kBF16 = kTileBF16, kF32 = kTileF32, kBytes = kTileBytes };

// (counter block layout: device/tile_collectives.cuh)
static constexpr int kMaxRanks = TCCL_MAX_RANKS;
static_assert(kMaxRanks == kTileCollMaxRanks, "rank limit of the API and of the device functions");

struct CollParams {
  int32_t op, dtype, rank, world_size, root;
  int32_t use_multimem;
  int32_t phase_mask;
  int32_t elem_size;   // bytes per element (scalar fallback granularity)
  uint32_t epoch;
  uint64_t src;        // local address (heap) of the input
  uint64_t dst;        // local address (heap) of the output (== src for in-place ops)
  uint64_t staging;    // one-shot all-reduce: local staging, two parity halves
  uint64_t stage_slot; // bytes between the halves (0: the message size rounded up to 16)
  uint64_t counters;   // local address of the counter block
  uint64_t mc_base;    // multicast alias of the heap (0 = none)
  uint64_t heap_base;  // this rank's heap base (to form multicast addresses)
  int64_t heap_stride;
  uint64_t bytes;      // payload per rank chunk (all-gather/scatter/reduce-scatter: chunk; else whole)
  uint64_t status;
  uint64_t budget_ns;
};

namespace {

__device__ __forceinline__ SymmWindow window_of(const CollParams& p) {
  SymmWindow w;
  w.base = p.heap_base - static_cast<uint64_t>(p.rank) * static_cast<uint64_t>(p.heap_stride);
  w.stride = static_cast<uint64_t>(p.heap_stride);
  w.mc_base = p.mc_base;
  w.rank = p.rank;
  w.world_size = p.world_size;
  return w;
}

__device__ __forceinline__ TileCollSync sync_of(const CollParams& p) {
  TileCollSync s;
  s.counters = reinterpret_cast<uint32_t*>(p.counters);
  s.epoch = p.epoch;
  s.status = reinterpret_cast<uint32_t*>(p.status);
  s.root = (p.op == kBroadcast || p.op == kScatter) ? p.root : -1;
  return s;
}

}  // namespace

// The launchable form of the device collectives in device/tile_collectives.cuh: the grid
// shares the data movement, one CTA runs the announcements and the final wait.
__global__ void __launch_bounds__(512) collective_kernel(const CollParams p) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  const SymmWindow w = window_of(p);
  const TileCollSync sync = sync_of(p);

  // ---- phase 1: announce ---------------------------------------------------
  // Everything this rank's stream did before the call is visible (kernel boundary).
  if ((p.phase_mask & 1) && blockIdx.x == 0) tile_coll_announce(w, sync);

  // ---- phase 2: wait for dependencies, move data, publish ------------------
  if (p.phase_mask & 2) {
    if (tile_coll_wait_ready(w, sync, wb)) {
      const TileCoop grid = tile_coop_grid();
      const bool mc = p.use_multimem != 0;
      void* src = reinterpret_cast<void*>(p.src);
      void* dst = reinterpret_cast<void*>(p.dst);
      switch (p.op) {
        case kAllGather: tile_allgather(w, src, dst, p.bytes, p.elem_size, mc, grid); break;
        case kBroadcast: tile_broadcast(w, dst, p.bytes, p.root, p.elem_size, mc, grid); break;
        case kScatter: tile_scatter(w, src, dst, p.bytes, p.root, p.elem_size, grid); break;
        case kReduceScatter: tile_reduce_scatter(w, src, dst, p.bytes, p.dtype, mc, grid); break;
        case kAllReduceTwoShot: tile_allreduce_chunk(w, dst, p.bytes, p.dtype, mc, grid); break;
        default: break;   // (kAllReduceOneShot moves its data in the dedicated kernel below)
      }
    }
    tile_coll_publish(w, sync, gridDim.x);
  }

  // ---- phase 3: wait for the completions this rank depends on --------------
  if ((p.phase_mask & 4) && blockIdx.x == 0) tile_coll_wait_done(w, sync, wb);
}

// One-shot all-reduce for small messages: every rank publishes a copy of its
// buffer in a staging slot (double-buffered by epoch parity, so no exit barrier
// is needed), then sums all ranks' copies straight into its own buffer.
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const CollParams p) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  const SymmWindow w = window_of(p);
  TileCollSync sync = sync_of(p);
  const uint64_t bytes = p.bytes;
  const uint64_t slot =
      p.stage_slot != 0 ? p.stage_slot : (bytes + 15) & ~static_cast<uint64_t>(15);
  char* stage = reinterpret_cast<char*>(p.staging + (p.epoch & 1u) * slot);
  char* buf = reinterpret_cast<char*>(p.dst);
  const TileCoop grid = tile_coop_grid();

  if (p.phase_mask & 1) {
    // publish a snapshot of the local buffer, then announce it (counters [0, 8): the
    // "ready" half of the block doubles as "snapshot published")
    coll_detail::copy_vec(stage, buf, bytes & ~static_cast<uint64_t>(15), 16, grid);
    if ((bytes & 15) && grid.tid == 0)
      for (uint64_t b = bytes & ~static_cast<uint64_t>(15); b < bytes; ++b) stage[b] = buf[b];
    // the last CTA to get here signals: same arrival counting as tile_coll_publish, but
    // on the "ready" counters
    __shared__ int is_last;
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      uint32_t* cta_done = sync.counters + 16;
      const uint32_t old = atomicAdd(cta_done, 1u);
      is_last = (old == gridDim.x - 1) ? 1 : 0;
      if (is_last) *cta_done = 0;
    }
    __syncthreads();
    if (is_last) {
      __threadfence_system();
      coll_detail::signal_set(w, sync, 0, -1);
    }
  }
  if (p.phase_mask & 2) {
    if (!coll_detail::wait_set(w, sync, 0, -1, wb, 64)) return;
    // the staged copies are one reduce-scatter chunk at offset 0 of every rank's slot
    coll_detail::reduce_chunk<false>(w, stage, buf, nullptr, 0, bytes, p.dtype, false, grid);
  }
}

// ---------------------------------------------------------------------------
// Pipelined relay broadcast for large messages on three or more ranks
// (device/tile_collectives.cuh: tile_relay_push / tile_relay_forward).  The handshake is
// the all-to-all one: every rank's buffer is written by the root and by the relays.
// phase_mask: 1 announce, 2 the root's push, 8 the relays' forwarding, 4 final wait; a
// launch normally runs all of them (15).  With ranks emulated on one GPU the host issues
// them one by one, the root's push before the relays' forwarding, so no launch waits for
// a later one.
// ---------------------------------------------------------------------------
struct RelayParams {
  int32_t rank, world_size, root, phase_mask;
  uint32_t epoch;
  uint64_t buf;          // local address of the tensor (same offset in every heap)
  uint64_t bytes;        // multiple of 16
  uint64_t piece_bytes;  // multiple of 16; ceil(bytes / piece_bytes) <= kTileRelayMaxPieces
  uint64_t flags;        // local address of the piece flags (uint32[kTileRelayMaxPieces])
  uint64_t counters;     // local address of the counter block
  uint64_t heap_base;
  int64_t heap_stride;
  uint64_t status, budget_ns;
};

__global__ void __launch_bounds__(512) broadcast_relay_kernel(const RelayParams p) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  SymmWindow w;
  w.base = p.heap_base - static_cast<uint64_t>(p.rank) * static_cast<uint64_t>(p.heap_stride);
  w.stride = static_cast<uint64_t>(p.heap_stride);
  w.mc_base = 0;
  w.rank = p.rank;
  w.world_size = p.world_size;
  TileCollSync sync;
  sync.counters = reinterpret_cast<uint32_t*>(p.counters);
  sync.epoch = p.epoch;
  sync.status = reinterpret_cast<uint32_t*>(p.status);
  sync.root = -1;                                    // all-to-all announcements and completions
  const bool is_root = p.rank == p.root;

  if ((p.phase_mask & 1) && blockIdx.x == 0) tile_coll_announce(w, sync);
  if (p.phase_mask & (is_root ? 2 : 8)) {
    if (tile_coll_wait_ready(w, sync, wb)) {
      void* buf = reinterpret_cast<void*>(p.buf);
      uint32_t* flags = reinterpret_cast<uint32_t*>(p.flags);
      if (is_root)
        tile_relay_push(w, buf, p.bytes, p.piece_bytes, flags, p.epoch, blockIdx.x, gridDim.x);
      else
        tile_relay_forward(w, buf, p.bytes, p.piece_bytes, p.root, flags, p.epoch, blockIdx.x,
                           gridDim.x, wb, sync.status);
    }
    tile_coll_publish(w, sync, gridDim.x);
  }
  if ((p.phase_mask & 4) && blockIdx.x == 0) tile_coll_wait_done(w, sync, wb);
}

// The same relay with bulk copies (cp.async.bulk) through shared memory instead of
// register copies: each of a CTA's four warps is an independent pipeline driven by its
// lane 0 (local memory -> 16 KiB slot -> peer).  A piece's flag is written when the bulk
// groups of THAT pipeline have completed, so publishing a piece waits for one pipeline's
// stores only; with register copies by 512 threads every flag needs a system-scope fence
// behind ALL of the CTA's stores, which on a loaded link waits for everything the SM has in
// flight (measured: 110 us for 16 MiB at 4 ranks against 24 us of wire time).  The flag is a
// RELEASE store at system scope behind cp.async.bulk.wait_group + fence.proxy.async: a
// completed bulk group is only promised to be visible to the thread that waited for it, and
// a relaxed flag was observed to overtake the data (512 MiB and 1 GiB broadcasts at 4 ranks
// forwarded stale pieces); the release makes the thread's completed writes visible system
// wide before the flag.
static constexpr int kRelayWarps = 4;
static constexpr int kRelaySlots = 2;
static constexpr uint32_t kRelaySlotBytes = 16 * 1024;
static constexpr uint32_t kRelaySmemBytes = kRelayWarps * kRelaySlots * kRelaySlotBytes;

__global__ void __launch_bounds__(kRelayWarps * 32) broadcast_relay_bulk_kernel(const RelayParams p) {
  extern __shared__ __align__(128) unsigned char relay_smem[];
  __shared__ __align__(8) uint64_t bars[kRelayWarps * kRelaySlots];
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) {
    abort_word = 0;
    for (int i = 0; i < kRelayWarps * kRelaySlots; ++i) mbar_init(smem_u32(&bars[i]), 1);
    mbar_fence_init();
  }
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  SymmWindow w;
  w.base = p.heap_base - static_cast<uint64_t>(p.rank) * static_cast<uint64_t>(p.heap_stride);
  w.stride = static_cast<uint64_t>(p.heap_stride);
  w.mc_base = 0;
  w.rank = p.rank;
  w.world_size = p.world_size;
  TileCollSync sync;
  sync.counters = reinterpret_cast<uint32_t*>(p.counters);
  sync.epoch = p.epoch;
  sync.status = reinterpret_cast<uint32_t*>(p.status);
  sync.root = -1;
  const bool is_root = p.rank == p.root;
  const int ws = p.world_size;

  if ((p.phase_mask & 1) && blockIdx.x == 0) tile_coll_announce(w, sync);
  if (p.phase_mask & (is_root ? 2 : 8)) {
    const bool ready = tile_coll_wait_ready(w, sync, wb);
    const int warp = threadIdx.x >> 5;
    if (ready && (threadIdx.x & 31) == 0) {
      char* buf = reinterpret_cast<char*>(p.buf);
      uint32_t* flags = reinterpret_cast<uint32_t*>(p.flags);
      const uint32_t my_smem = smem_u32(relay_smem) + warp * kRelaySlots * kRelaySlotBytes;
      const uint32_t my_bar = smem_u32(&bars[warp * kRelaySlots]);
      const uint32_t n_pieces = static_cast<uint32_t>((p.bytes + p.piece_bytes - 1) / p.piece_bytes);
      const uint32_t worker = blockIdx.x * kRelayWarps + warp;
      const uint32_t n_workers = gridDim.x * kRelayWarps;
      const uint32_t mine = static_cast<uint32_t>(p.rank < p.root ? p.rank : p.rank - 1);
      const uint32_t first = is_root ? worker : worker * (ws - 1) + mine;
      const uint32_t step = is_root ? n_workers : n_workers * (ws - 1);
      uint32_t use = 0;
      bool ok = true;
      for (uint32_t piece = first; ok && piece < n_pieces; piece += step) {
        const uint64_t p_off = static_cast<uint64_t>(piece) * p.piece_bytes;
        const uint64_t p_len = p.bytes - p_off < p.piece_bytes ? p.bytes - p_off : p.piece_bytes;
        char* to_root_relay = nullptr;
        if (is_root) {
          to_root_relay = coll_detail::peer_of(w, buf, relay_rank_of(piece, p.root, ws));
        } else {
          uint32_t seen = 0;
          if (!tile_wait_ge(flags + piece, p.epoch, wb, &seen)) {
            report_status(sync.status, kStatusTimeoutSignal, 66, p.epoch, seen, p.rank, piece);
            ok = false;
            break;
          }
          fence_proxy_async_all();     // the bulk loads below read what the flag covers
        }
        for (uint64_t off = p_off; ok && off < p_off + p_len; off += kRelaySlotBytes) {
          const uint32_t slot = use % kRelaySlots;
          const uint32_t phase = (use / kRelaySlots) & 1u;
          const uint64_t left = p_off + p_len - off;
          const uint32_t bytes = static_cast<uint32_t>(left < kRelaySlotBytes ? left : kRelaySlotBytes);
          // the stores that last read this slot (kRelaySlots uses ago) are done with it
          tma_store_wait_read<kRelaySlots - 1>();
          mbar_expect_tx(my_bar + 8 * slot, bytes);
          bulk_load(my_smem + slot * kRelaySlotBytes, buf + off, bytes, my_bar + 8 * slot);
          if (!mbar_wait(my_bar + 8 * slot, phase, wb)) {
            report_status(sync.status, kStatusTimeoutMbarrier, 67, 0, 0, p.rank, piece);
            ok = false;
            break;
          }
          if (is_root) {
            bulk_store(to_root_relay + off, my_smem + slot * kRelaySlotBytes, bytes);
          } else {
            for (int k = 1; k < ws; ++k) {               // peers staggered, the root left out
              const int r = (p.rank + k) % ws;
              if (r != p.root)
                bulk_store(coll_detail::peer_of(w, buf, r) + off, my_smem + slot * kRelaySlotBytes,
                           bytes);
            }
          }
          tma_store_commit();
          ++use;
        }
        if (is_root && ok) {
          tma_store_wait_all<0>();       // this pipeline's stores of the piece are complete
          fence_proxy_async_all();
          st_release_sys(coll_detail::peer_of(w, flags, relay_rank_of(piece, p.root, ws)) + piece,
                         p.epoch);
        }
      }
      tma_store_wait_all<0>();           // nothing of this pipeline still reads shared memory
      fence_proxy_async_all();
    }
    tile_coll_publish(w, sync, gridDim.x);
  }
  if ((p.phase_mask & 4) && blockIdx.x == 0) tile_coll_wait_done(w, sync, wb);
}

// ---------------------------------------------------------------------------
// Low-latency collectives (all-gather, broadcast, scatter, reduce-scatter) for small
// messages: data and flag travel in the same 16-byte store (device/tile_ll.cuh), so a call
// is one NVLink write latency plus one poll instead of announce / move / publish / wait.
// Reduce-scatter: every rank sends chunk d of its input to rank d and sums, in fp32 and in
// rank order, the lines it receives with its own chunk.  All-reduce (one-shot): every rank
// sends its whole vector to every peer and sums what it receives with its own, in place (a
// thread sends and later overwrites the same lines, so the send reads before the sum writes).
// ---------------------------------------------------------------------------
struct LLParams {
  int32_t op, dtype, rank, world_size, root, phase_mask;
  uint32_t epoch;        // 1, 2, 3 ... per call on this staging + counter block (also the flag)
  uint64_t src, dst;     // local addresses
  uint64_t stage;        // this rank's staging: [2 parities][n_slots][slot_bytes]
  uint64_t slot_bytes;   // staging per (parity, source): >= 2 * bytes
  int32_t n_slots;       // world_size (all-gather, reduce-scatter: one slot per source) or 1 (rooted ops)
  uint64_t counters;     // this rank's block: [0, 8) acknowledgements from rank d, [16] cta_done
  int64_t heap_stride;
  uint32_t bytes;        // payload per (source, destination), multiple of 8, <= kLLMaxBytes
  uint64_t status, budget_ns;
};

namespace {
// acc (4 floats for 16-bit types, 2 for fp32) += the 8 payload bytes {d0, d1}
__device__ __forceinline__ void ll_accumulate(int dtype, float* acc, uint32_t d0, uint32_t d1) {
  if (dtype == kF32) {
    acc[0] += __uint_as_float(d0);
    acc[1] += __uint_as_float(d1);
  } else if (dtype == kBF16) {
    const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d0));
    const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&d1));
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  } else {
    const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&d0));
    const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&d1));
    acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
  }
}
__device__ __forceinline__ uint2 ll_finish(int dtype, const float* acc) {
  uint2 o;
  if (dtype == kF32) {
    o.x = __float_as_uint(acc[0]);
    o.y = __float_as_uint(acc[1]);
  } else if (dtype == kBF16) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(acc[0], acc[1]);
    const __nv_bfloat162 b = __floats2bfloat162_rn(acc[2], acc[3]);
    o.x = *reinterpret_cast<const uint32_t*>(&a);
    o.y = *reinterpret_cast<const uint32_t*>(&b);
  } else {
    const __half2 a = __floats2half2_rn(acc[0], acc[1]);
    const __half2 b = __floats2half2_rn(acc[2], acc[3]);
    o.x = *reinterpret_cast<const uint32_t*>(&a);
    o.y = *reinterpret_cast<const uint32_t*>(&b);
  }
  return o;
}
}  // namespace

__global__ void __launch_bounds__(512) ll_copy_kernel(const LLParams p) {
  __shared__ uint32_t abort_word;
  __shared__ int failed, is_last;
  if (threadIdx.x == 0) { abort_word = 0; failed = 0; }
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  uint32_t* status = reinterpret_cast<uint32_t*>(p.status);
  uint32_t* counters = reinterpret_cast<uint32_t*>(p.counters);
  const int ws = p.world_size, rank = p.rank;
  const bool reducing = p.op == kReduceScatter || p.op == kAllReduceOneShot;
  const bool rooted = p.op != kAllGather && !reducing;
  const bool per_dest_chunk = p.op == kScatter || p.op == kReduceScatter;
  const bool sender = !rooted || rank == p.root;
  const bool receiver = !rooted || rank != p.root;
  const uint32_t parity = p.epoch & 1u;
  const uint64_t parity_off = static_cast<uint64_t>(parity) * p.n_slots * p.slot_bytes;
  const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x, nthreads = gridDim.x * blockDim.x;
  auto peer_addr = [&](uint64_t local, int r) {
    return local + static_cast<uint64_t>(static_cast<int64_t>(r - rank) * p.heap_stride);
  };

  if ((p.phase_mask & 1) && sender) {
    // The parity half about to be written was last used two calls ago: every receiver must
    // have acknowledged that call.
    if (p.epoch > 2) {
      const int d = threadIdx.x;
      if (d < ws && d != rank) {
        uint32_t seen = 0;
        if (!tile_wait_ge(counters + d, p.epoch - 2u, wb, &seen)) {
          report_status(status, kStatusTimeoutSignal, 70, p.epoch - 2u, seen, rank, d);
          failed = 1;
        }
      }
      __syncthreads();
    }
    if (!failed) {
      const int slot = rooted ? 0 : rank;
      for (int k = 1; k < ws; ++k) {
        const int d = (rank + k) % ws;
        const char* src = reinterpret_cast<const char*>(p.src) +
                          (per_dest_chunk ? static_cast<uint64_t>(d) * p.bytes : 0);
        char* lines = reinterpret_cast<char*>(peer_addr(p.stage, d)) + parity_off +
                      static_cast<uint64_t>(slot) * p.slot_bytes;
        ll_send(lines, src, p.bytes, p.epoch, tid, nthreads);
      }
      // this rank's own part never leaves the GPU
      if (p.op == kAllGather || p.op == kScatter) {
        const char* src = reinterpret_cast<const char*>(p.src) +
                          (p.op == kScatter ? static_cast<uint64_t>(rank) * p.bytes : 0);
        char* dst = reinterpret_cast<char*>(p.dst) +
                    (p.op == kAllGather ? static_cast<uint64_t>(rank) * p.bytes : 0);
        if (src != dst)
          for (uint32_t i = tid; i < (p.bytes >> 3); i += nthreads)
            reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(src)[i];
      }
    }
  }

  if ((p.phase_mask & 2) && receiver) {
    const char* stage = reinterpret_cast<const char*>(p.stage) + parity_off;
    bool ok = true;
    if (rooted) {
      ok = ll_recv(reinterpret_cast<char*>(p.dst), stage, p.bytes, p.epoch, tid, nthreads, wb);
    } else if (reducing) {
      const char* own = reinterpret_cast<const char*>(p.src) +
                        (per_dest_chunk ? static_cast<uint64_t>(rank) * p.bytes : 0);
      const uint32_t lines = p.bytes >> 3;
      for (uint32_t i = tid; i < lines && ok; i += nthreads) {
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        for (int s = 0; s < ws && ok; ++s) {          // rank order: same sum on every path
          uint32_t d0, d1;
          if (s == rank) {
            const uint2 v = *reinterpret_cast<const uint2*>(own + (static_cast<uint64_t>(i) << 3));
            d0 = v.x; d1 = v.y;
          } else {
            ok = ll_load_line(stage + static_cast<uint64_t>(s) * p.slot_bytes +
                                  static_cast<uint64_t>(i) * kLLLineBytes,
                              p.epoch, d0, d1, wb);
          }
          if (ok) ll_accumulate(p.dtype, acc, d0, d1);
        }
        if (ok)
          *reinterpret_cast<uint2*>(reinterpret_cast<char*>(p.dst) +
                                    (static_cast<uint64_t>(i) << 3)) = ll_finish(p.dtype, acc);
      }
    } else {
      for (int k = 1; k < ws && ok; ++k) {
        const int s = (rank + ws - k) % ws;
        ok = ll_recv(reinterpret_cast<char*>(p.dst) + static_cast<uint64_t>(s) * p.bytes,
                     stage + static_cast<uint64_t>(s) * p.slot_bytes, p.bytes, p.epoch, tid,
                     nthreads, wb);
      }
    }
    if (!ok) report_status(status, kStatusTimeoutSignal, 71, p.epoch, 0, rank, 0);
    // Acknowledge once every CTA of this launch has consumed its lines.
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(counters + 16, 1u);
      is_last = (old == gridDim.x - 1) ? 1 : 0;
      if (is_last) counters[16] = 0;
    }
    __syncthreads();
    if (is_last) {
      const int s = threadIdx.x;
      if (s < ws && s != rank && (!rooted || s == p.root))
        red_release_sys_add(reinterpret_cast<uint32_t*>(peer_addr(p.counters, s)) + rank, 1u);
    }
  }
}

}  // namespace tileccl

using namespace tileccl;

extern "C" int tccl_collective_ll_launch(int32_t op, int32_t dtype, int32_t rank,
                                         int32_t world_size, int32_t root,
                                         int32_t phase_mask, uint32_t epoch, uint64_t src,
                                         uint64_t dst, uint64_t stage, uint64_t counters,
                                         int64_t heap_stride, uint64_t bytes,
                                         uint64_t slot_bytes, int32_t grid,
                                         uint64_t status, uint64_t budget_ns, uint64_t stream) {
  TCCL_CHECK_ARG(op == kAllGather || op == kBroadcast || op == kScatter || op == kReduceScatter ||
                     op == kAllReduceOneShot,
                 "the low-latency path serves all-gather, broadcast, scatter, reduce-scatter and "
                 "one-shot all-reduce");
  TCCL_CHECK_ARG((op != kReduceScatter && op != kAllReduceOneShot) || dtype == kF16 ||
                     dtype == kBF16 || dtype == kF32,
                 "a reduction needs a float dtype (0 fp16, 1 bf16, 2 fp32)");
  TCCL_CHECK_ARG(world_size >= 2 && world_size <= kMaxRanks, "world_size must be 2..8");
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size && root >= 0 && root < world_size, "bad rank/root");
  TCCL_CHECK_ARG(bytes > 0 && bytes <= kLLMaxBytes && bytes % 8 == 0,
                 "low-latency messages are multiples of 8 bytes, at most " << kLLMaxBytes);
  TCCL_CHECK_ARG(src % 8 == 0 && dst % 8 == 0 && stage % 16 == 0 && stage != 0 && counters != 0,
                 "buffers must be 8-byte aligned and staging / counters present");
  TCCL_CHECK_ARG(epoch != 0, "epoch starts at 1");
  TCCL_CHECK_ARG(slot_bytes >= kLLMinSlotBytes && slot_bytes % 16 == 0 && slot_bytes >= 2 * bytes,
                 "a staging slot holds 2 bytes per payload byte, at least " << kLLMinSlotBytes);
  TCCL_CHECK_ARG(grid >= 1 && grid <= 64, "grid must be 1..64");
  LLParams p;
  p.op = op; p.dtype = dtype; p.rank = rank; p.world_size = world_size; p.root = root;
  p.phase_mask = phase_mask;
  p.epoch = epoch; p.src = src; p.dst = dst; p.stage = stage; p.slot_bytes = slot_bytes;
  p.n_slots = (op == kAllGather || op == kReduceScatter || op == kAllReduceOneShot) ? world_size : 1;
  p.counters = counters; p.heap_stride = heap_stride; p.bytes = static_cast<uint32_t>(bytes);
  p.status = status; p.budget_ns = budget_ns ? budget_ns : 2000000000ull;
  ll_copy_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  TCCL_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int tccl_broadcast_relay_launch(int32_t rank, int32_t world_size, int32_t root,
                                           int32_t phase_mask, uint32_t epoch, uint64_t buf,
                                           uint64_t bytes, uint64_t piece_bytes, uint64_t flags,
                                           uint64_t counters, uint64_t heap_base,
                                           int64_t heap_stride, int32_t grid, int32_t bulk,
                                           uint64_t status, uint64_t budget_ns, uint64_t stream) {
  TCCL_CHECK_ARG(world_size >= 3 && world_size <= kMaxRanks, "the relay broadcast needs 3..8 ranks");
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size && root >= 0 && root < world_size, "bad rank/root");
  TCCL_CHECK_ARG(buf != 0 && buf % 16 == 0 && bytes > 0 && bytes % 16 == 0,
                 "buffer and size must be multiples of 16 bytes");
  TCCL_CHECK_ARG(piece_bytes >= 16 && piece_bytes % 16 == 0, "piece size must be a multiple of 16");
  TCCL_CHECK_ARG((bytes + piece_bytes - 1) / piece_bytes <= kTileRelayMaxPieces,
                 "at most " << kTileRelayMaxPieces << " pieces per call");
  TCCL_CHECK_ARG(flags != 0 && counters != 0 && epoch != 0, "flags, counters and an epoch >= 1");
  TCCL_CHECK_ARG(grid >= 1, "grid must be >= 1");
  RelayParams p;
  p.rank = rank; p.world_size = world_size; p.root = root; p.phase_mask = phase_mask;
  p.epoch = epoch; p.buf = buf; p.bytes = bytes; p.piece_bytes = piece_bytes; p.flags = flags;
  p.counters = counters; p.heap_base = heap_base; p.heap_stride = heap_stride; p.status = status;
  p.budget_ns = budget_ns ? budget_ns : 2000000000ull;
  if (bulk) {
    static std::atomic<int> configured[64];
    int dev = 0;
    TCCL_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev >= 0 && dev < 64 && !configured[dev].load(std::memory_order_acquire)) {
      TCCL_CHECK_CUDA(cudaFuncSetAttribute(broadcast_relay_bulk_kernel,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>(kRelaySmemBytes)));
      configured[dev].store(1, std::memory_order_release);
    }
    broadcast_relay_bulk_kernel<<<grid, kRelayWarps * 32, kRelaySmemBytes,
                                  reinterpret_cast<cudaStream_t>(stream)>>>(p);
  } else {
    broadcast_relay_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  }
  TCCL_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int tccl_collective_launch(int32_t op, int32_t dtype, int32_t rank, int32_t world_size,
                                      int32_t root, int32_t use_multimem, int32_t phase_mask,
                                      int32_t elem_size, uint32_t epoch, uint64_t src, uint64_t dst, uint64_t staging,
                                      uint64_t stage_slot, uint64_t counters, uint64_t mc_base, uint64_t heap_base,
                                      int64_t heap_stride, uint64_t bytes, int32_t grid,
                                      uint64_t status, uint64_t budget_ns, uint64_t stream) {
  TCCL_CHECK_ARG(op >= kAllGather && op <= kScatter, "unknown collective");
  TCCL_CHECK_ARG(world_size >= 1 && world_size <= kMaxRanks, "world_size must be 1..8");
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size && root >= 0 && root < world_size, "bad rank/root");
  TCCL_CHECK_ARG(counters != 0, "missing counter block");
  TCCL_CHECK_ARG(grid >= 1, "grid must be >= 1");
  TCCL_CHECK_ARG(elem_size == 1 || elem_size == 2 || elem_size == 4 || elem_size == 8,
                 "elem_size must be 1, 2, 4 or 8");
  TCCL_CHECK_ARG(bytes % elem_size == 0, "byte count is not a whole number of elements");
  TCCL_CHECK_ARG((src % 16) == 0 && (dst % 16) == 0, "buffers must be 16-byte aligned");
  if (use_multimem) TCCL_CHECK_ARG(mc_base != 0, "multimem requested without a multicast mapping");
  if (op == kAllGather || op == kScatter || op == kReduceScatter)
    TCCL_CHECK_ARG(world_size == 1 || bytes % 16 == 0 || !use_multimem,
                   "multimem path needs 16-byte multiple chunks");
  CollParams p;
  p.op = op; p.dtype = dtype; p.rank = rank; p.world_size = world_size; p.root = root;
  p.use_multimem = use_multimem; p.phase_mask = phase_mask; p.epoch = epoch;
  p.elem_size = elem_size;
  p.src = src; p.dst = dst; p.staging = staging; p.stage_slot = stage_slot;
  p.counters = counters; p.mc_base = mc_base;
  p.heap_base = heap_base; p.heap_stride = heap_stride; p.bytes = bytes; p.status = status;
  p.budget_ns = budget_ns ? budget_ns : 2000000000ull;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  if (op == kAllReduceOneShot) {
    TCCL_CHECK_ARG(staging != 0, "one-shot all-reduce needs a staging buffer");
    TCCL_CHECK_ARG(stage_slot == 0 || (stage_slot % 16 == 0 && stage_slot >= bytes),
                   "stage_slot must be a multiple of 16 and hold the message");
    allreduce_oneshot_kernel<<<grid, 512, 0, s>>>(p);
  } else {
    collective_kernel<<<grid, 512, 0, s>>>(p);
  }
  TCCL_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

// ---------------------------------------------------------------------------
// All-reduce without any allocation (see collectives_noalloc.h for the contract)
// ---------------------------------------------------------------------------
#include "collectives_noalloc.h"

// Scratch of the no-allocation entry point: lives in the library image, one copy
// per GPU that loads the library.  Rank r of a call uses the block at r *
// TCCL_NOALLOC_RANK_BYTES: [staging parity 0][staging parity 1][counter block].
// In host code this name is only a handle for cudaGetSymbolAddress, never an address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[TCCL_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kNoAllocMaxDevices = 64;
// Device address of the array per device ordinal; filled on first use.  Atomic: two host
// threads may make their first call on a device at the same time (both then resolve the
// same address, which is harmless).
std::atomic<void*> g_noalloc_scratch_ptr[kNoAllocMaxDevices];
}  // namespace

extern "C" int tccl_allreduce_sum_noalloc(const uint64_t* buffers, int32_t n_ranks, int32_t dtype,
                                          uint64_t count, uint64_t stream) {
  TCCL_CHECK_ARG(buffers != nullptr, "buffers is null");
  TCCL_CHECK_ARG(n_ranks >= 1 && n_ranks <= TCCL_NOALLOC_MAX_RANKS,
                 "n_ranks must be 1.." << TCCL_NOALLOC_MAX_RANKS << ", got " << n_ranks);
  TCCL_CHECK_ARG(dtype == kF16 || dtype == kBF16 || dtype == kF32,
                 "dtype must be 0 (fp16), 1 (bf16) or 2 (fp32)");
  const uint64_t elem = dtype == kF32 ? 4 : 2;
  TCCL_CHECK_ARG(count > 0, "count must be positive");
  // Compare before multiplying: count * elem wraps for absurd counts.
  TCCL_CHECK_ARG(count <= TCCL_NOALLOC_MAX_BYTES / elem,
                 "message of " << count << " elements exceeds the built-in scratch ("
                               << TCCL_NOALLOC_MAX_BYTES << " bytes per buffer); use the heap-based "
                               << "all-reduce for larger messages");
  const uint64_t bytes = count * elem;
  TCCL_CHECK_ARG(bytes <= TCCL_NOALLOC_MAX_BYTES,
                 "message of " << bytes << " bytes exceeds the built-in scratch ("
                               << TCCL_NOALLOC_MAX_BYTES << " bytes per buffer); use the heap-based "
                               << "all-reduce for larger messages");
  for (int r = 0; r < n_ranks; ++r)
    TCCL_CHECK_ARG(buffers[r] != 0 && buffers[r] % 16 == 0,
                   "buffer " << r << " must be a non-null, 16-byte aligned device address");
  int dev = 0;
  TCCL_CHECK_CUDA(cudaGetDevice(&dev));
  TCCL_CHECK_ARG(dev >= 0 && dev < kNoAllocMaxDevices, "device ordinal out of range");
  void* scratch_ptr = g_noalloc_scratch_ptr[dev].load(std::memory_order_acquire);
  if (scratch_ptr == nullptr) {
    // Once per device, with that device current: the device address of the array.
    TCCL_CHECK_CUDA(cudaGetSymbolAddress(&scratch_ptr, g_noalloc_scratch));
    TCCL_CHECK_ARG(scratch_ptr != nullptr, "cudaGetSymbolAddress returned a null scratch address");
    g_noalloc_scratch_ptr[dev].store(scratch_ptr, std::memory_order_release);
  }
  const uint64_t scratch = reinterpret_cast<uint64_t>(scratch_ptr);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  // The counters keep the previous call's values: they must start at zero.
  for (int r = 0; r < n_ranks; ++r)
    TCCL_CHECK_CUDA(cudaMemsetAsync(
        reinterpret_cast<void*>(scratch + r * uint64_t(TCCL_NOALLOC_RANK_BYTES) +
                                2 * uint64_t(TCCL_NOALLOC_MAX_BYTES)),
        0, 256, s));
  int grid = static_cast<int>((bytes / 16 + 1023) / 1024);
  grid = grid < 1 ? 1 : (grid > 32 ? 32 : grid);
  // phase 1 for every rank (publish a snapshot), then phase 2 for every rank (sum):
  // kernels of one GPU never wait on one another.
  for (int phase = 1; phase <= 2; ++phase) {
    for (int r = 0; r < n_ranks; ++r) {
      CollParams p;
      p.op = kAllReduceOneShot; p.dtype = dtype; p.rank = r; p.world_size = n_ranks; p.root = 0;
      p.use_multimem = 0; p.phase_mask = phase; p.elem_size = static_cast<int32_t>(elem);
      p.epoch = 1;
      p.src = buffers[r]; p.dst = buffers[r];
      p.staging = scratch + r * uint64_t(TCCL_NOALLOC_RANK_BYTES);
      p.stage_slot = TCCL_NOALLOC_MAX_BYTES;
      p.counters = p.staging + 2 * uint64_t(TCCL_NOALLOC_MAX_BYTES);
      p.mc_base = 0; p.heap_base = 0;
      p.heap_stride = TCCL_NOALLOC_RANK_BYTES;
      p.bytes = bytes; p.status = 0; p.budget_ns = 2000000000ull;
      allreduce_oneshot_kernel<<<grid, 512, 0, s>>>(p);
      TCCL_CHECK_CUDA(cudaGetLastError());
    }
  }
  return kOk;
}

TILECCL_DEFINE_DEBUG_READER(tccl_debug_read_collectives)

namespace tileccl {
cudaError_t preload_collective_kernels() {
  cudaFuncAttributes a;
  cudaError_t e = cudaFuncGetAttributes(&a, collective_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, allreduce_oneshot_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, ll_copy_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, broadcast_relay_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, broadcast_relay_bulk_kernel);
  return e;
}
}  // namespace tileccl
