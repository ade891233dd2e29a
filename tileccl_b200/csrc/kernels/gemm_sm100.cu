// Persistent warp-specialised tcgen05 GEMM for sm_100a, with the collective
// that follows it fused into the epilogue.
//
// Two forms of one kernel (template parameter kPair):
//   one CTA per tile   128 x 256 tile, tcgen05.mma.cta_group::1, four-stage operand ring.
//                      Used for tile-range launches (emulated ranks, host-streamed operand)
//                      and traced launches.
//   CTA pair per tile  a cluster of two CTAs on a 256 x 256 tile, tcgen05.mma.cta_group::2:
//                      every CTA stages its own 128 rows of A and 128 of the 256 columns of
//                      B (32 KB instead of 48 KB per K block and SM), six stages; the
//                      leader CTA issues the MMAs, commits are multicast to both CTAs'
//                      barriers, each CTA owns the accumulator and the epilogue of its 128
//                      rows.  Used whenever a launch runs the rank's whole tile order.
//
// Roles per CTA (256 threads):
//   warp 0      TMA producer: A / B tiles -> shared-memory ring (local memory only, no
//               multicast); for the own tiles of a reduce-scatter also the peers' staged
//               partial tiles, which the tensor cores add to the accumulator (identity x
//               tile)
//   warp 1      MMA issuer (fp32 accumulators in TMEM, two 256-column buffers)
//   warp 2, 3   TMEM allocation; all-gather push of the A operand; communication warps of
//               the `stores` / `multimem` push modes; incoming-TileGroup waiter
//   warps 4..7  epilogue: tcgen05.ld -> (SiLU-gate) -> cast -> swizzled staging in shared
//               memory -> TMA store to the local destination and, per mode, TMA stores into
//               the peers' memory, followed by an add on the peers' TileGroup counters.
//
// What replaces what in the reference: the plain mode is its persistent GEMM
// (tileccl/kernels/gemm.py:52-167); push-all is the GEMM-output all-gather
// (tileccl/ops.py:1700-1790, a host loop of torch.mm + tile all-gather there);
// reduce-scatter is tileccl/ops.py:1793-1896; all-scatter is the wg_specialized
// pattern (tileccl/patterns/wg_specialized.py:210-352) with the communication role
// played by the epilogue warps instead of dedicated SMs.
//
// Peer traffic is stores only (TMA store, plain st.global, or multimem.st);
// operands are always TMA-loaded from this GPU's own memory, without multicast.
#include "gemm_sm100.cuh"

#include "../device/ptx.cuh"
#include "../device/tile_compute.cuh"
#include "../device/tile_sync.cuh"
#include "../plan/tile_order.h"

namespace tileccl {

namespace {

struct TileCoord {
  int a_row0, b_col0;   // operand coordinates
  int out_x, out_y;     // destination-local coordinates (elements)
  int owner;            // reduce-scatter: rank that owns the tile; else this rank
  int lm;               // tile row inside the owner's sub-problem (TileGroup = lm / group_m_tiles)
  bool valid;           // false: padding half of the last pair-tile row
};

// One-CTA kernel: `t` indexes the rank's 128-row tiles.  CTA-pair kernel: `t` indexes
// 256-row pair-tiles (same visiting order over half as many tile rows) and CTA `cta` of
// the pair owns tile row 2 * (pair row) + cta, which may lie past the last real tile row
// (`valid` = false: the CTA still takes part in the MMA but stores and signals nothing).
template <bool kPair>
__device__ __forceinline__ TileCoord decode_tile(const FusedGemmParams& p, int t, int cta = 0) {
  const int m_rows = kPair ? (p.m_tiles_local + 1) / 2 : p.m_tiles_local;
  const TileOrderShape shape{m_rows, p.n_tiles_local, p.owners, p.rank, p.world_size,
                             kPair ? p.rot_m_tiles / 2 : p.rot_m_tiles,
                             kPair ? (p.rs_own_lag + 1) / 2 : p.rs_own_lag};
  TileOrderEntry e = tile_order_decode(shape, t);
  if (kPair) e.lm = e.lm * 2 + cta;
  TileCoord c;
  c.valid = e.lm < p.m_tiles_local;
  c.owner = e.owner;
  c.lm = e.lm;
  c.a_row0 = e.lm * kBM;
  c.b_col0 = e.ln * kBN;
  if (p.owners > 1) {
    if (p.split_axis == 0) c.a_row0 += c.owner * p.a_rows_per_owner;
    else c.b_col0 += c.owner * p.b_cols_per_owner;
  }
  c.out_y = e.lm * kBM;
  c.out_x = p.epi_op == kEpiSiluGate ? e.ln * (kBN / 2) : e.ln * kBN;
  return c;
}

__device__ __forceinline__ uint32_t* peer_counter(const FusedGemmParams& p, int dest_rank,
                                                  int src_slot, int group) {
  int64_t a = static_cast<int64_t>(p.sig_local) +
              static_cast<int64_t>(dest_rank - p.rank) * p.heap_stride;
  return reinterpret_cast<uint32_t*>(a) + src_slot * p.sig_stride + group;
}

// m-tiles in TileGroup g of a sub-problem with `m_tiles` tile rows.
__device__ __forceinline__ int group_m_count(const FusedGemmParams& p, int g) {
  int left = p.m_tiles_local - g * p.group_m_tiles;
  return left < p.group_m_tiles ? left : p.group_m_tiles;
}

__device__ __forceinline__ void tma_store_3d(const CUtensorMap* m, int x, int y, int z,
                                             uint32_t smem_src) {
  asm volatile(
      "cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::
          "l"(reinterpret_cast<uint64_t>(m)),
      "r"(x), "r"(y), "r"(z), "r"(smem_src)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t smem_dst, const CUtensorMap* m, int x, int y,
                                            int z, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_3d_pair(uint32_t smem_dst, const CUtensorMap* m, int x,
                                                 int y, int z, uint32_t cluster_bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.tile"
      ".mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(smem_dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y), "r"(z), "r"(cluster_bar)
      : "memory");
}

// Shared-memory geometry of the two kernel forms.  One CTA: 128 x 256 tile, 48 KB per K
// block, four stages.  CTA pair (tcgen05 cta_group::2): 256 x 256 per pair, every CTA stages
// its own 128 rows of A and 128 of the 256 columns of B (32 KB), six stages.
#ifndef TCCL_PAIR_STAGES
#define TCCL_PAIR_STAGES 6
#endif
#ifndef TCCL_PAIR_EPI_BUFS
#define TCCL_PAIR_EPI_BUFS 2
#endif
// Tiles by which a TileGroup signal trails the bulk stores it announces.  One tile: by the
// time the next tile's stores have been issued the previous tile's have almost always
// landed, and a reduce-scatter owner learns of its partial tiles a tile earlier than with
// two (measured: reduce-scatter 3 - 9 % faster at 2 and 8 GPUs, all-gather unchanged).
#ifndef TCCL_SIGNAL_DELAY_TILES
#define TCCL_SIGNAL_DELAY_TILES 1
#endif
static constexpr int kPend = TCCL_SIGNAL_DELAY_TILES;

// kBounce (CTA pairs only): one operand stage is given up for a 32 KB bounce ring through
// which warps 2 and 3 push the all-gathered A operand to the peers as bulk copies.
static constexpr int kBounceSlotBytes = 8192;
static constexpr int kBounceSlotsPerWarp = 2;

template <bool kPair, bool kBounce = false>
struct Geo {
  static_assert(kPair || !kBounce, "the bounce ring exists in the CTA-pair form only");
  static constexpr int kNumStages = kPair ? (kBounce ? TCCL_PAIR_STAGES - 1 : TCCL_PAIR_STAGES)
                                          : kStages;
  static constexpr int kBounceBytes = kBounce ? 2 * kBounceSlotsPerWarp * kBounceSlotBytes : 0;
  // staging buffers per epilogue warp: a deeper ring lets the epilogue run further ahead of
  // bulk stores that the link has not taken yet
  static constexpr int kEpi = kPair ? TCCL_PAIR_EPI_BUFS : kEpiBufs;
  static constexpr int kBBytes = kPair ? kStageBBytes / 2 : kStageBBytes;
  static constexpr int kBytes = kStageABytes + kBBytes;
  static constexpr int kBBoxes = kPair ? kBN / 2 / 64 : kBN / 64;   // 64-column boxes of an MN-major B
  static constexpr int kPipeBytes = kNumStages * kBytes;
  static_assert(kPipeBytes + kEpiWarps * kEpi * kEpiBufBytes + kBounceBytes <= kSmemPipe + kSmemEpi,
                "operand ring + staging + bounce ring exceed their shared-memory budget");
};

}  // namespace

template <bool kPair, bool kBounce>
__global__ void __launch_bounds__(kThreads, 1)
fused_gemm_sm100_kernel(const __grid_constant__ FusedGemmParams p) {
  using G = Geo<kPair, kBounce>;
  constexpr int kNS = G::kNumStages;
  extern __shared__ uint8_t smem_raw[];
  const uint64_t t_entry = p.trace != 0 ? globaltimer_ns() : 0;
  // 128-byte swizzled tiles need 1024-byte aligned bases.
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t smem_epi = smem_base + G::kPipeBytes;
  const uint32_t smem_ctl = smem_base + kSmemPipe + kSmemEpi;
  uint8_t* ctl_generic = smem_raw + (smem_ctl - smem_u32(smem_raw));

  // In the pair form every CTA has all barriers; the leader's "full" and "accumulator
  // empty" barriers are the ones in use (both CTAs report to them), "empty" and
  // "accumulator full" are signalled in both CTAs by multicast commits.
  const uint32_t bar_full = smem_ctl;                         // kNS x 8 B
  const uint32_t bar_empty = bar_full + 8 * kNS;              // kNS x 8 B
  const uint32_t bar_acc_full = bar_empty + 8 * kNS;          // kAccBufs x 8 B
  const uint32_t bar_acc_empty = bar_acc_full + 8 * kAccBufs; // kAccBufs x 8 B
  const uint32_t bar_drain = bar_acc_empty + 8 * kAccBufs;    // 8 B
  const uint32_t tmem_slot = bar_drain + 8;                   // 4 B
  volatile uint32_t* tmem_slot_g =
      reinterpret_cast<volatile uint32_t*>(ctl_generic + (tmem_slot - smem_ctl));
  volatile uint32_t* abort_flag = tmem_slot_g + 1;
  // Slabs (one per epilogue warp and tile) whose local bulk stores have completed; the
  // communication warps poll it to learn which tiles of C they may forward.
  const uint32_t done_count = tmem_slot + 8;
  volatile uint32_t* done_count_g = tmem_slot_g + 2;
  static_assert(8 * (2 * kNS + 2 * kAccBufs + 1) + 16 <= 200, "control block overflow");
  // Tile-index ring of the dynamic scheduler: the scheduling thread (TMA producer; in a
  // pair the leader's) publishes positions of the tile order, every other role consumes them.
  constexpr int kSched = 4;
  const uint32_t bar_sched_full = smem_ctl + 256;                    // kSched x 8 B
  const uint32_t bar_sched_empty = bar_sched_full + 8 * kSched;      // kSched x 8 B
  const uint32_t sched_tile = bar_sched_empty + 8 * kSched;          // kSched x 4 B
  static_assert(256 + 16 * kSched + 4 * kSched <= kSmemCtl, "control block overflow");
  const uint32_t smem_bounce = smem_epi + kEpiWarps * G::kEpi * kEpiBufBytes;
  const uint32_t bar_bounce = smem_ctl + 200;                 // 2 warps x 2 slots x 8 B
  static_assert(200 + 8 * 2 * kBounceSlotsPerWarp <= kSmemCtl, "control block overflow");

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int cta = kPair ? static_cast<int>(cluster_ctarank()) : 0;   // 0 = leader of the pair
  const bool leader = cta == 0;
  uint32_t* status = reinterpret_cast<uint32_t*>(p.status);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kNS; ++s) {
      mbar_init(bar_full + 8 * s, 1);
      mbar_init(bar_empty + 8 * s, 1);
    }
    for (int a = 0; a < kAccBufs; ++a) {
      mbar_init(bar_acc_full + 8 * a, 1);
      mbar_init(bar_acc_empty + 8 * a, kPair ? 2 * kEpiWarps : kEpiWarps);
    }
    mbar_init(bar_drain, 1);
    for (int i = 0; i < kSched; ++i) {
      mbar_init(bar_sched_full + 8 * i, 1);
      // readers of a slot: MMA thread + four epilogue warps, in a pair those of both CTAs
      // (the peer's TMA producer reads in place of its idle MMA thread)
      mbar_init(bar_sched_empty + 8 * i, kPair ? 2 * (1 + kEpiWarps) : 1 + kEpiWarps);
    }
    if (kBounce)
      for (int i = 0; i < 2 * kBounceSlotsPerWarp; ++i) mbar_init(bar_bounce + 8 * i, 1);
    *abort_flag = 0;
    *done_count_g = 0;
    for (int i = 0; i < kStatPerCta; ++i)
      asm volatile("st.shared.u64 [%0], %1;" ::"r"(smem_ctl + 352 + 8 * i), "l"(0ull) : "memory");
    mbar_fence_init();
  }
  if (warp == 2) {
    if (kPair) {
      tmem_alloc_pair(tmem_slot, kAccBufs * kBN);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(tmem_slot, kAccBufs * kBN);
      tmem_relinquish();
    }
  }
  tcgen05_fence_before();
  __syncthreads();
  if (kPair) cluster_sync_all();   // barriers and TMEM of both CTAs exist
  tcgen05_fence_after();
  const uint32_t tmem_base = *tmem_slot_g;

  WaitBudget wb;
  wb.start(p.wait_budget_ns, abort_flag);
  // Trace layout: uint64[tile slots][4 epilogue warps][4] followed by uint64[CTAs][8]
  // (kernel entry / roles start / incoming TileGroups seen / after the final CTA barrier /
  // epilogue warp 0..3 done, i.e. its last bulk store complete and last signal sent).
  uint64_t* const trace_tiles = reinterpret_cast<uint64_t*>(p.trace);
  uint64_t* const trace_cta =
      p.trace == 0 ? nullptr
                   : trace_tiles + static_cast<int64_t>(p.trace_tile_slots) * (kEpiWarps * 4) +
                         static_cast<int64_t>(blockIdx.x) * 8;
  if (trace_cta != nullptr && threadIdx.x == 0) {
    trace_cta[0] = t_entry;
    trace_cta[1] = globaltimer_ns();
  }

  // Tile iteration: 128-row tiles per CTA, or 256-row pair-tiles per CTA pair (the pair
  // form always runs the rank's whole tile order).
  const int first = kPair ? static_cast<int>(blockIdx.x >> 1)
                          : p.tile_begin + static_cast<int>(blockIdx.x);
  const int step = kPair ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int tile_end =
      kPair ? ((p.m_tiles_local + 1) / 2) * p.n_tiles_local * p.owners : p.tile_end;
  // Finished tiles of C are forwarded to the peers by warps 2 and 3 (16-byte stores or
  // multimem stores read back from this rank's copy of C) rather than by the epilogue.
  const bool comm_push = p.world_size > 1 && p.push_mode != kPushTma &&
                         (p.mode == kModePushAll || p.mode == kModeAllScatter);

  // Per-call counters (FusedGemmParams::stats): each role keeps its own sums in registers and
  // adds them once, when it is done.
  // (Sums go to shared memory first; one thread per CTA adds the CTA's totals to its own row
  // of the global table when the CTA retires.  Global atomics from the roles themselves
  // measured 10 - 40 us on a reduce-scatter call.)
  const uint32_t stat_smem = smem_ctl + 352;          // 4 x 8 B
  static_assert(352 + 8 * kStatPerCta <= kSmemCtl, "control block overflow");
  auto stat_add = [&](int word, uint64_t v) {
    if (p.stats != 0 && v != 0)
      asm volatile("red.shared.add.u64 [%0], %1;" ::"r"(stat_smem + 8 * word), "l"(v) : "memory");
  };

  // ---------------------------- dynamic tile scheduling ----------------------------
  // SMs do not get equal shares of the link, so with a fixed round-robin assignment the
  // slowest SMs finish long after the others (and a reduce-scatter owner waits for the
  // slowest pusher of every TileGroup).  Here positions of the tile order are handed out
  // one at a time from a global counter instead.
  const bool dyn = p.sched_counter != 0 && !comm_push;
  // Scheduling thread: publish position `t` (-1 = no more tiles) as the n-th entry.
  auto sched_publish = [&](uint32_t n, int t) -> bool {
    const uint32_t slot = n % kSched, ph = (n / kSched) & 1u;
    if (!mbar_wait(bar_sched_empty + 8 * slot, ph ^ 1u, wb)) return false;
    st_shared_cluster_u32(kPair ? mapa_shared(sched_tile + 4 * slot, 0) : sched_tile + 4 * slot,
                          static_cast<uint32_t>(t));
    if (kPair) {
      st_shared_cluster_u32(mapa_shared(sched_tile + 4 * slot, 1), static_cast<uint32_t>(t));
      mbar_arrive_cluster(mapa_shared(bar_sched_full + 8 * slot, 0));
      mbar_arrive_cluster(mapa_shared(bar_sched_full + 8 * slot, 1));
    } else {
      mbar_arrive(bar_sched_full + 8 * slot);
    }
    return true;
  };
  // Any other role (one thread per role): the n-th entry; -2 when the wait gave up.
  auto sched_consume = [&](uint32_t n) -> int {
    const uint32_t slot = n % kSched, ph = (n / kSched) & 1u;
    for (uint32_t it = 0;; ++it) {
      if (mbar_try_wait_cluster(bar_sched_full + 8 * slot, ph)) break;
      if (wb.expired(it)) { *abort_flag = 1; return -2; }
    }
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(sched_tile + 4 * slot) : "memory");
    if (kPair) mbar_arrive_cluster(mapa_shared(bar_sched_empty + 8 * slot, 0));
    else mbar_arrive(bar_sched_empty + 8 * slot);
    return static_cast<int>(v);
  };
  auto sched_fetch = [&]() -> int {
    const uint32_t v = atomicAdd(reinterpret_cast<uint32_t*>(p.sched_counter), 1u);
    return v < static_cast<uint32_t>(tile_end) ? static_cast<int>(v) : -1;
  };

  // Entry handshake (see FusedGemmParams::entry_local).  Warp-collective: lane d polls
  // peer d's "entered" word; returns false (status 45) when a peer never shows up.
  auto wait_peers_entered = [&]() -> bool {
    if (p.entry_local == 0 || p.world_size <= 1) return true;
    bool ok_lane = true;
    if (lane < p.world_size && lane != p.rank) {
      uint32_t seen = 0;
      if (!tile_wait_ge(reinterpret_cast<const uint32_t*>(p.entry_local) + lane, p.epoch, wb,
                        &seen)) {
        report_status(status, kStatusTimeoutSignal, 45, p.epoch, seen, p.rank, lane);
        *abort_flag = 1;
        ok_lane = false;
      }
    }
    return __all_sync(0xffffffffu, ok_lane);
  };
  auto announce_entry = [&]() {
    if (p.entry_local == 0 || !p.announce_entry || p.world_size <= 1 || blockIdx.x != 0) return;
    if (lane < p.world_size && lane != p.rank)
      red_release_sys_add(
          reinterpret_cast<uint32_t*>(static_cast<int64_t>(p.entry_local) +
                                      static_cast<int64_t>(lane - p.rank) * p.heap_stride) + p.rank,
          1u);
  };

  // ------------------------- communication warps (2, 3) -------------------------
  // Warp 2 forwards rows [0, 64) of every finished tile, warp 3 rows [64, 128): one
  // warp-wide 16-byte load per tile row from this rank's C (still in L2), one store per
  // peer (or one multimem store), eight rows in flight.  The fence + counter update
  // that publishes the half tile stalls only this warp, never the epilogue.
  auto comm_role = [&](int half) {
    const int tile_cols = p.epi_op == kEpiSiluGate ? kBN / 2 : kBN;
    const int vpr = tile_cols / 8;   // 16-byte vectors per tile row
    const int rpi = 32 / vpr;        // tile rows covered by one warp-wide access
    const int lrow = lane / vpr, lvec = lane % vpr;
    uint32_t n_tiles = 0;
    if (!wait_peers_entered()) return;
    for (int t = first; t < tile_end; t += step) {
      ++n_tiles;
      const uint32_t want = n_tiles * kEpiWarps;
      bool got = true;
      uint32_t seen = 0;
      for (uint32_t it = 0;; ++it) {
        asm volatile("ld.acquire.cta.shared.u32 %0, [%1];" : "=r"(seen) : "r"(done_count) : "memory");
        if (seen >= want) break;
        if (wb.expired(it)) { got = false; break; }
        if (it > 8) __nanosleep(64);
      }
      got = __all_sync(0xffffffffu, got);
      if (!got) {
        if (lane == 0 && !wb.aborted())
          report_status(status, kStatusTimeoutMbarrier, 60 + half, want, seen, p.rank, t);
        break;
      }
      fence_proxy_async_all();
      const TileCoord c = decode_tile<kPair>(p, t, cta);
      if (!c.valid) continue;
      int lo = c.out_x, hi = c.out_x + tile_cols;
      if (hi > p.out_cols) hi = p.out_cols;
      if (p.mode == kModeAllScatter) {
        if (lo < p.scatter_col_begin) lo = p.scatter_col_begin;
        if (hi > p.scatter_col_end) hi = p.scatter_col_end;
      }
      if (hi > lo) {
        const int col = c.out_x + lvec * 8;
        const bool col_ok = col >= lo && col < hi;
        const int y0 = c.out_y + half * (kBM / 2) + lrow;
        const int64_t col_off = static_cast<int64_t>(col) * 2;
        const char* src = reinterpret_cast<const char*>(p.out_ptr[p.rank]);
        for (int r0 = 0; r0 < kBM / 2; r0 += 8 * rpi) {
          uint4 v[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int row = y0 + r0 + j * rpi;
            if (col_ok && row < p.out_rows)
              v[j] = ld_remote_v4(src + static_cast<int64_t>(row) * p.out_ld_bytes + col_off);
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int row = y0 + r0 + j * rpi;
            if (!(col_ok && row < p.out_rows)) continue;
            const int64_t off = static_cast<int64_t>(row) * p.out_ld_bytes + col_off;
            if (p.push_mode == kPushMultimem) {
              multimem_st_v4(reinterpret_cast<char*>(p.out_mc_ptr) + off, v[j]);
            } else {
              for (int d = 1; d < p.world_size; ++d)
                st_remote_v4(reinterpret_cast<char*>(p.out_ptr[(p.rank + d) % p.world_size]) + off,
                             v[j]);
            }
          }
        }
      }
      if (p.sig_local != 0) {
        fence_acq_rel_sys();   // every lane's peer stores are performed before the signal
        __syncwarp();
        if (lane == 0) {
          const int group = c.lm / p.group_m_tiles;
          for (int d = 1; d < p.world_size; ++d)
            red_release_sys_add(peer_counter(p, (p.rank + d) % p.world_size, p.rank, group),
                                static_cast<uint32_t>(kEpiWarps / 2));
        }
      }
    }
  };

  // ------------------- all-gather push of the A operand (warps 2, 3) -------------------
  // This rank's shard goes to the same place in every peer's heap: 16-byte stores, or one
  // multimem store per 16 bytes when a multicast mapping is given.  A warp sustains well
  // under 1 GB/s of remote stores, so both spare warps of every CTA share the work; each
  // adds one arrival to the peers' gate counter when its part has been performed.
  auto ag_push_role = [&](int part) {
    if (p.ag_bytes == 0 || !p.do_ag_push || p.world_size <= 1) return;
    if (!wait_peers_entered()) return;
    if (kBounce) {
      // Bulk copies through the bounce ring: local shard -> shared memory -> peer, 8 KB at a
      // time, two slots per warp.  Destinations go in the order rank-1, rank-2, ...: a
      // consumer visits the shards in the order own, rank+1, rank+2, ..., so at every moment
      // each rank receives the shard it needs next from exactly one sender.  A destination's
      // gate counter is raised as soon as this warp's part for it has landed.
      if (lane != 0) return;
      const char* src = reinterpret_cast<const char*>(p.ag_src);
      const uint64_t n_chunks = (p.ag_bytes + kBounceSlotBytes - 1) / kBounceSlotBytes;
      const uint32_t my_smem = smem_bounce + part * kBounceSlotsPerWarp * kBounceSlotBytes;
      const uint32_t my_bar = bar_bounce + part * kBounceSlotsPerWarp * 8;
      uint32_t use = 0;
      bool ok = true;
      for (int k = 1; ok && k < p.world_size; ++k) {
        const int dest = (p.rank - k + p.world_size) % p.world_size;
        char* dst = reinterpret_cast<char*>(static_cast<int64_t>(p.ag_dst) +
                                            static_cast<int64_t>(dest - p.rank) * p.heap_stride);
        for (uint64_t c = static_cast<uint64_t>(blockIdx.x) * 2 + part; c < n_chunks;
             c += static_cast<uint64_t>(gridDim.x) * 2) {
          const uint32_t slot = use % kBounceSlotsPerWarp;
          const uint32_t phase = (use / kBounceSlotsPerWarp) & 1u;
          const uint64_t off = c * kBounceSlotBytes;
          const uint32_t bytes = static_cast<uint32_t>(
              p.ag_bytes - off < kBounceSlotBytes ? p.ag_bytes - off : kBounceSlotBytes);
          // the store that last read this slot (kBounceSlotsPerWarp uses ago) is done with it
          tma_store_wait_read<kBounceSlotsPerWarp - 1>();
          mbar_expect_tx(my_bar + 8 * slot, bytes);
          bulk_load(my_smem + slot * kBounceSlotBytes, src + off, bytes, my_bar + 8 * slot);
          if (!mbar_wait(my_bar + 8 * slot, phase, wb)) {
            report_status(status, kStatusTimeoutMbarrier, 13, 0, 0, p.rank, static_cast<uint32_t>(c));
            ok = false;
            break;
          }
          bulk_store(dst + off, my_smem + slot * kBounceSlotBytes, bytes);
          tma_store_commit();
          ++use;
        }
        tma_store_wait_all<0>();          // this warp's part for `dest` has landed
        fence_proxy_async_all();
        if (ok)
          red_release_sys_add(
              reinterpret_cast<uint32_t*>(static_cast<int64_t>(p.a_gate) +
                                          static_cast<int64_t>(dest - p.rank) * p.heap_stride) +
                  p.rank,
              1u);
      }
      return;
    }
    constexpr int U = 8;
    const char* src = reinterpret_cast<const char*>(p.ag_src);
    const uint64_t nvec = p.ag_bytes >> 4;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * 2 * 32;
    uint64_t i = (static_cast<uint64_t>(blockIdx.x) * 2 + part) * 32 + lane;
    for (; i < nvec; i += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int j = 0; j < U; ++j)
        if (i + j * stride < nvec) v[j] = ld_stream_v4(src + ((i + j * stride) << 4));
#pragma unroll
      for (int j = 0; j < U; ++j) {
        if (i + j * stride >= nvec) continue;
        const uint64_t off = (i + j * stride) << 4;
        if (p.ag_mc_dst != 0) {
          multimem_st_v4(reinterpret_cast<char*>(p.ag_mc_dst) + off, v[j]);
        } else {
          for (int d = 1; d < p.world_size; ++d) {
            const int r = (p.rank + d) % p.world_size;
            st_remote_v4(reinterpret_cast<char*>(static_cast<int64_t>(p.ag_dst) +
                                                 static_cast<int64_t>(r - p.rank) * p.heap_stride) +
                             off, v[j]);
          }
        }
      }
    }
    fence_acq_rel_sys();
    __syncwarp();
    if (lane == 0) {
      for (int d = 1; d < p.world_size; ++d) {
        const int r = (p.rank + d) % p.world_size;
        red_release_sys_add(
            reinterpret_cast<uint32_t*>(static_cast<int64_t>(p.a_gate) +
                                        static_cast<int64_t>(r - p.rank) * p.heap_stride) + p.rank,
            1u);
      }
    }
  };

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (elect_one_sync()) {
      tma_prefetch_desc(&p.tma_a);
      tma_prefetch_desc(&p.tma_b);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      // The position for the next tile is fetched one tile ahead: the atomic's round trip
      // (about a microsecond) then hides behind this tile's K loop instead of delaying it.
      int t_next = (dyn && leader) ? sched_fetch() : -1;
      uint64_t peer_wait_clk = 0, n_tiles_done = 0;   // (the SM cycle counter: a %globaltimer
                                                      // read costs about a microsecond)
      for (uint32_t n_seq = 0; ok; ++n_seq) {
        int t;
        if (dyn) {
          if (leader) {
            t = t_next;
            if (!sched_publish(n_seq, t)) {
              report_status(status, kStatusTimeoutMbarrier, 14, 0, 0, p.rank, n_seq);
              ok = false;
              break;
            }
            if (t >= 0) t_next = sched_fetch();
          } else {
            t = sched_consume(n_seq);
          }
          if (t < 0) break;
        } else {
          t = first + static_cast<int>(n_seq) * step;
          if (t >= tile_end) break;
        }
        const TileCoord c = decode_tile<kPair>(p, t, cta);
        n_tiles_done += kPair ? 2 : 1;
        if (p.a_gate != 0 && c.valid) {
          // Rows of A written by a peer: wait for that peer's arrival counter.
          int src = c.a_row0 / p.a_gate_rows_per_rank;
          if (src != p.rank) {
            uint32_t seen = 0;
            const long long w0 = clock64();
            const bool arrived = tile_wait_ge(reinterpret_cast<const uint32_t*>(p.a_gate) + src,
                                              p.a_gate_target, wb, &seen);
            peer_wait_clk += static_cast<uint64_t>(clock64() - w0);
            if (!arrived) {
              report_status(status, kStatusTimeoutSignal, 10, p.a_gate_target, seen, p.rank, t);
              *abort_flag = 1;
              ok = false;
              break;
            }
          }
        }
        for (int kb = 0; kb < p.k_blocks; ++kb) {
          if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, wb)) {
            report_status(status, kStatusTimeoutMbarrier, 11, 0, 0, p.rank, t);
            ok = false;
            break;
          }
          const uint32_t sa = smem_base + stage * G::kBytes;
          const uint32_t sb = sa + kStageABytes;
          if (kPair) {
            // Own halves; the bytes of both CTAs are counted on the leader's barrier.
            if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * G::kBytes);
            const uint32_t bar = mapa_shared(bar_full + 8 * stage, 0);
            const int b_col = c.b_col0 + cta * (kBN / 2);
            tma_load_2d_pair(sa, &p.tma_a, kb * kBK, c.a_row0, bar);
            if (p.b_kmajor) {
              tma_load_2d_pair(sb, &p.tma_b_half, kb * kBK, b_col, bar);
            } else {
#pragma unroll
              for (int i = 0; i < G::kBBoxes; ++i)
                tma_load_2d_pair(sb + i * (64 * kBK * 2), &p.tma_b_half, b_col + i * 64, kb * kBK,
                                 bar);
            }
          } else {
            const uint32_t bar = bar_full + 8 * stage;
            mbar_expect_tx(bar, G::kBytes);
            tma_load_2d(sa, &p.tma_a, kb * kBK, c.a_row0, bar);
            if (p.b_kmajor) {
              tma_load_2d(sb, &p.tma_b, kb * kBK, c.b_col0, bar);
            } else {
#pragma unroll
              for (int i = 0; i < G::kBBoxes; ++i)
                tma_load_2d(sb + i * (64 * kBK * 2), &p.tma_b, c.b_col0 + i * 64, kb * kBK, bar);
            }
          }
          if (++stage == kNS) { stage = 0; phase ^= 1u; }
        }
        if (ok && p.mode == kModeReduceScatter && p.world_size > 1 && c.owner == p.rank) {
          // Own tile: after its K blocks, the peers' staged partial tiles go through the
          // same pipeline, in rank order, next to the identity.  One CTA: two 64-row
          // halves of the tile.  CTA pair: the 256 x 256 identity times the two stacked
          // tiles of the pair, K' = 256 in four blocks; this CTA's rows of the identity are
          // zero outside its own two blocks (loaded as out-of-range boxes), and it stages
          // its 128 columns of both tiles.
          const int lm_first = kPair ? c.lm - cta : c.lm;
          const int n_rows = kPair ? 2 : 1;
          for (int i = 0; ok && i < n_rows; ++i) {
            const int lm = lm_first + i;
            if (lm >= p.m_tiles_local) continue;
            const int group = lm / p.group_m_tiles;
            const uint32_t target =
                p.epoch * static_cast<uint32_t>((p.world_size - 1) * group_m_count(p, group) *
                                                p.n_tiles_local * kEpiWarps);
            uint32_t seen = 0;
            const long long w0 = clock64();
            const bool arrived = tile_wait_ge(reinterpret_cast<const uint32_t*>(p.sig_local) + group,
                                              target, wb, &seen);
            peer_wait_clk += static_cast<uint64_t>(clock64() - w0);
            if (!arrived) {
              report_status(status, kStatusTimeoutSignal, 40, target, seen, p.rank, group);
              *abort_flag = 1;
              ok = false;
            }
          }
          if (!ok) break;
          fence_proxy_async_all();   // bulk reads of the partials come after that observation
          constexpr int kRedBlocks = (kPair ? 2 : 1) * (kBM / kBK);
          for (int src = 0; ok && src < p.world_size; ++src) {
            if (src == p.rank) continue;
            const int z = p.stage_parity * p.world_size + src;
            for (int hb = 0; hb < kRedBlocks; ++hb) {
              if (!mbar_wait(bar_empty + 8 * stage, phase ^ 1u, wb)) {
                report_status(status, kStatusTimeoutMbarrier, 12, 0, 0, p.rank, t);
                ok = false;
                break;
              }
              const uint32_t sa = smem_base + stage * G::kBytes;
              const uint32_t sb = sa + kStageABytes;
              if (kPair) {
                if (leader) mbar_expect_tx(bar_full + 8 * stage, 2 * G::kBytes);
                const uint32_t bar = mapa_shared(bar_full + 8 * stage, 0);
                tma_load_2d_pair(sa, &p.tma_ident, (hb - 2 * cta) * kBK, 0, bar);
                const int y = lm_first * kBM + hb * kBK;     // row of the stacked pair of tiles
#pragma unroll
                for (int i = 0; i < G::kBBoxes; ++i)
                  tma_load_3d_pair(sb + i * (64 * kBK * 2), &p.tma_stage,
                                   c.out_x + cta * (kBN / 2) + i * 64, y, z, bar);
              } else {
                const uint32_t bar = bar_full + 8 * stage;
                mbar_expect_tx(bar, G::kBytes);
                tma_load_2d(sa, &p.tma_ident, hb * kBK, 0, bar);
#pragma unroll
                for (int i = 0; i < G::kBBoxes; ++i)
                  tma_load_3d(sb + i * (64 * kBK * 2), &p.tma_stage, c.out_x + i * 64,
                              c.out_y + hb * kBK, z, bar);
              }
              if (++stage == kNS) { stage = 0; phase ^= 1u; }
            }
          }
        }
      }
      stat_add(2, peer_wait_clk);
      stat_add(3, leader ? n_tiles_done : 0);
      if (!ok) {
        // Let loads that are still in flight land before the CTA retires.
        for (int s = 0; s < kNS; ++s)
          for (int it = 0; it < 100000 && !mbar_try_wait(bar_full + 8 * s, 0) &&
                           !mbar_try_wait(bar_full + 8 * s, 1); ++it) {}
      }
    }
  } else if (warp == 1 && leader) {
    // ------------------- MMA issuer (in a pair: the leader CTA only) -------------------
    if (elect_one_sync()) {
      constexpr int kM = kPair ? 2 * kBM : kBM;
      const uint32_t idesc = umma_idesc_f16(p.is_bf16, 0, p.b_kmajor ? 0 : 1, kM, kBN);
      const uint32_t idesc_red = umma_idesc_f16(p.is_bf16, 0, 1, kM, kBN);
      auto mma = [&](uint32_t d, uint64_t da, uint64_t db, uint32_t id, uint32_t accum) {
        if (kPair) umma_f16_pair(d, da, db, id, accum); else umma_f16(d, da, db, id, accum);
      };
      // One arrival on `bar` (in both CTAs of a pair) once the MMAs issued so far are done.
      auto commit = [&](uint32_t bar) {
        if (kPair) umma_commit_pair(bar, 3); else umma_commit(bar);
      };
      uint32_t stage = 0, phase = 0;
      uint32_t acc = 0, acc_phase = 0;
      bool ok = true;
      for (uint32_t n_seq = 0; ok; ++n_seq) {
        int t;
        if (dyn) {
          t = sched_consume(n_seq);
          if (t < 0) break;
        } else {
          t = first + static_cast<int>(n_seq) * step;
          if (t >= tile_end) break;
        }
        if (!mbar_wait(bar_acc_empty + 8 * acc, acc_phase ^ 1u, wb)) {
          report_status(status, kStatusTimeoutMbarrier, 20, 0, 0, p.rank, t);
          ok = false;
          break;
        }
        tcgen05_fence_after();
        const uint32_t d_tmem = tmem_base + acc * kBN;
        // Own reduce-scatter tiles continue with the peers' partial tiles (see the producer).
        const bool reduce_tile = p.mode == kModeReduceScatter && p.world_size > 1 &&
                                 decode_tile<kPair>(p, t, cta).owner == p.rank;
        const int kb_total =
            p.k_blocks +
            (reduce_tile ? (kPair ? 2 : 1) * (kBM / kBK) * (p.world_size - 1) : 0);
        for (int kb = 0; kb < kb_total; ++kb) {
          if (!mbar_wait(bar_full + 8 * stage, phase, wb)) {
            report_status(status, kStatusTimeoutMbarrier, 21, kb_total, kb, p.rank, t);
            ok = false;
            break;
          }
          tcgen05_fence_after();
          const uint32_t sa = smem_base + stage * G::kBytes;
          const uint32_t sb = sa + kStageABytes;
#pragma unroll
          for (int k = 0; k < kBK / kUmmaK; ++k) {
            const uint64_t da = umma_smem_desc_sw128(sa + k * (kUmmaK * 2), 16, 1024);
            // A staged partial tile is always an MN-major ([K', N] row-major) B operand.
            const bool b_k = p.b_kmajor && kb < p.k_blocks;
            const uint64_t db =
                b_k ? umma_smem_desc_sw128(sb + k * (kUmmaK * 2), 16, 1024)
                    : umma_smem_desc_sw128(sb + k * (kUmmaK * 128), 64 * kBK * 2, 1024);
            mma(d_tmem, da, db, b_k == (p.b_kmajor != 0) ? idesc : idesc_red,
                (kb | k) != 0 ? 1u : 0u);
          }
          commit(bar_empty + 8 * stage);  // frees the stage once these MMAs have read it
          if (++stage == kNS) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        commit(bar_acc_full + 8 * acc);   // accumulator complete -> epilogue
        if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
      }
      if (!ok) {
        // Outstanding MMAs must finish before TMEM is released.
        if (kPair) umma_commit_pair(bar_drain, 1); else umma_commit(bar_drain);
        for (int it = 0; it < 1000000 && !mbar_try_wait(bar_drain, 0); ++it) {}
      }
    }
  } else if (warp == 2) {
    announce_entry();
    ag_push_role(0);
    if (comm_push) comm_role(0);
  } else if (warp == 3) {
    ag_push_role(1);
    if (comm_push) comm_role(1);
    // ---------------------- incoming TileGroup waiter -------------------------
    if (p.mode == kModePushAll && p.wait_incoming && p.world_size > 1) {
      const int groups = (p.m_tiles_local + p.group_m_tiles - 1) / p.group_m_tiles;
      const int total = p.world_size * groups;
      const uint32_t* sig = reinterpret_cast<const uint32_t*>(p.sig_local);
      for (int i = blockIdx.x * 32 + lane; i < total; i += gridDim.x * 32) {
        const int src = i / groups, g = i - src * groups;
        if (src == p.rank) continue;
        const uint32_t target =
            p.epoch * static_cast<uint32_t>(group_m_count(p, g) * p.n_tiles_local * kEpiWarps);
        uint32_t seen = 0;
        const long long w0 = clock64();
        const bool arrived = tile_wait_ge(sig + src * p.sig_stride + g, target, wb, &seen);
        stat_add(2, static_cast<uint64_t>(clock64() - w0));
        if (!arrived) {
          report_status(status, kStatusTimeoutSignal, 30, target, seen, p.rank, i);
          break;
        }
      }
      __syncwarp();
      if (trace_cta != nullptr && lane == 0) trace_cta[2] = globaltimer_ns();
    }
  } else if (warp >= 4) {
    // -------------------------------- epilogue --------------------------------
    const int q = warp - 4;                       // TMEM lane quarter and 32-row slab
    const bool bf16 = p.is_bf16 != 0;
    const uint32_t my_epi = smem_epi + q * (G::kEpi * kEpiBufBytes);
    uint8_t* my_epi_g = smem_raw + (my_epi - smem_u32(smem_raw));
    const int n_chunks = p.epi_op == kEpiSiluGate ? (kBN / 2) / kChunkN : kBN / kChunkN;
    uint32_t acc = 0, acc_phase = 0;
    uint32_t buf = 0;
    bool ok = true;
    // Peer copies issued by this warp (bulk stores) must not start before the peers have
    // entered this call; checked once, right before the first of them.
    uint64_t bytes_pushed = 0, signals_sent = 0;     // lane 0 only
    bool peers_entered = !(p.world_size > 1 && p.push_mode == kPushTma && p.entry_local != 0 &&
                           (p.mode == kModePushAll || p.mode == kModeAllScatter));
    // lane 0: the last kPend tiles whose signals have not been sent yet ([0] = oldest)
    bool pend_valid[kPend] = {};
    bool slab_pending = false;   // lane 0: a slab whose completion the comm warps still await
    int pend_owner[kPend] = {}, pend_group[kPend] = {};
    auto any_pending = [&]() {
      bool any = false;
#pragma unroll
      for (int i = 0; i < kPend; ++i) any = any || pend_valid[i];
      return any;
    };
    // One release-add per destination: "one more slab of TileGroup `g` from this rank has landed".
    auto send_signal = [&](int owner, int g, bool after_bulk) {
      const bool relaxed = after_bulk && (p.tuning & kTuneRelaxedSignalAfterBulk) != 0;
      auto add = [&](uint32_t* ctr) {
        ++signals_sent;
        if (relaxed)
          asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(ctr), "r"(1u) : "memory");
        else
          red_release_sys_add(ctr, 1u);
      };
      if (p.mode == kModeReduceScatter) {
        add(peer_counter(p, owner, 0, g));
      } else {
        for (int d = 1; d < p.world_size; ++d)
          add(peer_counter(p, (p.rank + d) % p.world_size, p.rank, g));
      }
    };
    for (uint32_t n_seq = 0; ok; ++n_seq) {
      int t;
      if (dyn) {
        t = 0;
        if (lane == 0) t = sched_consume(n_seq);
        t = __shfl_sync(0xffffffffu, t, 0);
        if (t < 0) break;
      } else {
        t = first + static_cast<int>(n_seq) * step;
        if (t >= tile_end) break;
      }
      const TileCoord c = decode_tile<kPair>(p, t, cta);
      const int group = c.lm / p.group_m_tiles;
      const bool reduce_here = p.mode == kModeReduceScatter && c.owner == p.rank;

      if (reduce_here && p.world_size > 1 && lane == 0 && any_pending() &&
          !mbar_try_wait(bar_acc_full + 8 * acc, acc_phase)) {
        // The accumulator of an own tile may be held up until the peers' partial tiles have
        // arrived (the producer warp waits for them).  Signals this warp still holds back
        // for earlier remote tiles go out before it blocks: the peers' owners wait for them
        // just as this rank waits for theirs, and holding them would close a cycle.
        tma_store_wait_all<0>();
        fence_proxy_async_all();
#pragma unroll
        for (int i = 0; i < kPend; ++i) {
          if (pend_valid[i]) send_signal(pend_owner[i], pend_group[i], true);
          pend_valid[i] = false;
        }
      }

      if (!mbar_wait(bar_acc_full + 8 * acc, acc_phase, wb)) {
        if (lane == 0) report_status(status, kStatusTimeoutMbarrier, 41, 0, 0, p.rank, t);
        ok = false;
        break;
      }
      tcgen05_fence_after();
      if (p.trace != 0 && lane == 0)
        trace_tiles[(static_cast<int64_t>(kPair ? 2 * t + cta : t) * kEpiWarps + q) * 4] = globaltimer_ns();
      const uint32_t t_acc = tmem_base + acc * kBN + (static_cast<uint32_t>(q * 32) << 16);

      for (int ch = 0; ch < n_chunks; ++ch) {
        float v[kChunkN];
        {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_acc + ch * kChunkN, r0);
          tmem_ld_32x32b_x32(t_acc + ch * kChunkN + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = __uint_as_float(r0[i]);
            v[32 + i] = __uint_as_float(r1[i]);
          }
        }
        if (p.epi_op == kEpiSiluGate) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32b_x32(t_acc + kBN / 2 + ch * kChunkN, r0);
          tmem_ld_32x32b_x32(t_acc + kBN / 2 + ch * kChunkN + 32, r1);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            v[i] = apply_elementwise(kOpSilu, v[i]) * __uint_as_float(r0[i]);
            v[32 + i] = apply_elementwise(kOpSilu, v[32 + i]) * __uint_as_float(r1[i]);
          }
        }
        if (ch == n_chunks - 1) {
          // Every TMEM read of this accumulator is done: hand it back to the MMA warp.
          tcgen05_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (kPair) mbar_arrive_cluster(mapa_shared(bar_acc_empty + 8 * acc, 0));
            else mbar_arrive(bar_acc_empty + 8 * acc);
          }
        }

        const int col0 = c.out_x + ch * kChunkN;     // destination-local column of v[0]
        // Staging buffer `buf` was last read by the stores committed two chunks ago.
        if (lane == 0) tma_store_wait_read<G::kEpi - 1>();
        __syncwarp();
        const uint32_t sbuf = my_epi + buf * kEpiBufBytes;
#pragma unroll
        for (int j = 0; j < kChunkN / 8; ++j) {
          const uint4 w = tile_cast_f32x8(bf16, &v[j * 8]);
          const uint32_t addr = sbuf + lane * 128 + ((j ^ (lane & 7)) << 4);
          asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(w.x), "r"(w.y),
                       "r"(w.z), "r"(w.w)
                       : "memory");
        }
        fence_proxy_async_smem();
        __syncwarp();

        const int y = c.out_y + q * kSlabM;
        bool push_all = p.mode == kModePushAll;
        if (p.mode == kModeAllScatter)
          push_all = col0 >= p.scatter_col_begin && col0 < p.scatter_col_end;

        if (p.mode == kModeReduceScatter && !reduce_here) {
          // Partial tile -> owner's staging slot for (parity, this rank).
          const int z = p.stage_parity * p.world_size + p.rank;
          if (p.push_mode == kPushTma) {
            if (lane == 0) {
              tma_store_3d(&p.tma_out[c.owner], col0, y, z, sbuf);
              bytes_pushed += kEpiBufBytes;
            }
          } else {
            char* dst = reinterpret_cast<char*>(p.out_ptr[c.owner]) +
                        static_cast<int64_t>(z) * p.out_slot_bytes;
            const uint8_t* sg = my_epi_g + buf * kEpiBufBytes;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int idx = lane + 32 * i, r = idx >> 3, j = idx & 7;
              if (y + r < p.out_rows && col0 + j * 8 < p.out_cols) {
                const uint4 w = *reinterpret_cast<const uint4*>(sg + r * 128 + ((j ^ (r & 7)) << 4));
                st_remote_v4(dst + static_cast<int64_t>(y + r) * p.out_ld_bytes +
                                 static_cast<int64_t>(col0 + j * 8) * 2, w);
              }
            }
          }
        } else {
          // Local destination (plain GEMM, own all-gather rows, reduced tile).
          const int local_slot = p.mode == kModeGemm ? 0 : p.rank;
          if (lane == 0) tma_store_3d(&p.tma_out[local_slot], col0, y, 0, sbuf);
          // Peer copies: one bulk store per destination here, or (other push modes) left
          // to the communication warps, which forward the tile once it is complete.
          if (push_all && p.world_size > 1 && p.push_mode == kPushTma) {
            if (!peers_entered) {
              if (!wait_peers_entered()) {
                ok = false;
                if (lane == 0) tma_store_commit();   // the local store issued above
                break;
              }
              peers_entered = true;
            }
            if (lane == 0) {
              for (int d = 1; d < p.world_size; ++d)
                tma_store_3d(&p.tma_out[(p.rank + d) % p.world_size], col0, y, 0, sbuf);
              bytes_pushed += static_cast<uint64_t>(p.world_size - 1) * kEpiBufBytes;
            }
          }
        }
        if (lane == 0) tma_store_commit();
        buf = (buf + 1u) % G::kEpi;
      }
      if (!ok) break;

      if (p.trace != 0 && lane == 0)
        trace_tiles[(static_cast<int64_t>(kPair ? 2 * t + cta : t) * kEpiWarps + q) * 4 + 1] = globaltimer_ns();
      // ---- TileGroup signalling: this slab of this tile is now on its way ----
      const bool signals = c.valid && p.world_size > 1 && p.sig_local != 0 &&
                           (p.mode == kModePushAll || p.mode == kModeAllScatter ||
                            (p.mode == kModeReduceScatter && !reduce_here));
      if (comm_push) {
        // Tell the communication warps that the previous tile's slab is in global memory
        // (its bulk groups have completed; this tile's may still be in flight).
        if (lane == 0) {
          if (slab_pending) {
            if (n_chunks == 4) tma_store_wait_all<4>(); else tma_store_wait_all<2>();
            fence_proxy_async_all();
            asm volatile("red.release.cta.shared.add.u32 [%0], 1;" ::"r"(done_count) : "memory");
          }
          slab_pending = true;
        }
      } else if (p.push_mode == kPushTma) {
        // Peer copies are bulk stores issued by lane 0.  The signal of a tile is sent kPend
        // tiles late: by then its bulk groups have (almost always) completed, i.e. the data has
        // reached the peer, while the groups of the most recent kPend tiles are still in
        // flight, so neither the NVLink round trip nor the queueing behind other SMs' stores
        // stalls this warp.
        if (lane == 0) {
          if (pend_valid[0]) {
            if (n_chunks == 4) tma_store_wait_all<4 * kPend>(); else tma_store_wait_all<2 * kPend>();
            fence_proxy_async_all();
            if (p.trace != 0)
              trace_tiles[(static_cast<int64_t>(kPair ? 2 * t + cta : t) * kEpiWarps + q) * 4 + 2] =
                  globaltimer_ns();
            send_signal(pend_owner[0], pend_group[0], true);
          }
#pragma unroll
          for (int i = 0; i + 1 < kPend; ++i) {
            pend_valid[i] = pend_valid[i + 1];
            pend_owner[i] = pend_owner[i + 1];
            pend_group[i] = pend_group[i + 1];
          }
          pend_valid[kPend - 1] = signals;
          pend_owner[kPend - 1] = c.owner;
          pend_group[kPend - 1] = group;
        }
      } else if (signals) {
        if (lane == 0) tma_store_wait_all<0>();   // the local bulk store
        fence_proxy_async_all();
        fence_acq_rel_sys();                      // every lane's peer stores are ordered first
        __syncwarp();
        if (lane == 0) send_signal(c.owner, group, false);
      }
      // Plain GEMM feeding a consumer kernel on the same GPU (producer / consumer
      // pattern): publish the slab on this rank's own TileGroup counter.
      if (p.mode == kModeGemm && p.sig_local != 0 && c.valid) {
        if (lane == 0) tma_store_wait_all<0>();
        fence_proxy_async_all();
        __threadfence();
        __syncwarp();
        if (lane == 0)
          red_release_sys_add(reinterpret_cast<uint32_t*>(p.sig_local) + group, 1u);
      }
      if (p.trace != 0 && lane == 0)
        trace_tiles[(static_cast<int64_t>(kPair ? 2 * t + cta : t) * kEpiWarps + q) * 4 + 3] = globaltimer_ns();

      if (++acc == kAccBufs) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) {
      tma_store_wait_all<0>();
      fence_proxy_async_all();
      if (slab_pending)
        asm volatile("red.release.cta.shared.add.u32 [%0], 1;" ::"r"(done_count) : "memory");
#pragma unroll
      for (int i = 0; i < kPend; ++i)
        if (pend_valid[i]) send_signal(pend_owner[i], pend_group[i], true);
      if (trace_cta != nullptr) trace_cta[4 + q] = globaltimer_ns();
      stat_add(0, bytes_pushed);
      stat_add(1, signals_sent);
    }
  }

  // In a pair neither CTA may retire while its partner can still read its operands or
  // touch its barriers; TMEM goes back only after every MMA and TMEM read is done.
  tcgen05_fence_before();
  __syncthreads();
  if (trace_cta != nullptr && threadIdx.x == 0) trace_cta[3] = globaltimer_ns();
  if (p.stats != 0 && threadIdx.x == 0) {
    uint64_t* row = reinterpret_cast<uint64_t*>(p.stats) +
                    static_cast<int64_t>(blockIdx.x) * kStatPerCta;
    for (int i = 0; i < kStatPerCta; ++i) {
      uint64_t v;
      asm volatile("ld.shared.u64 %0, [%1];" : "=l"(v) : "r"(stat_smem + 8 * i) : "memory");
      if (v != 0) row[i] += v;           // one writer per row; launches are stream-ordered
    }
  }
  if (p.sched_counter != 0 && threadIdx.x == 0) {
    // The last CTA to get here leaves the scheduler's counters at zero for the next launch.
    uint32_t* sc = reinterpret_cast<uint32_t*>(p.sched_counter);
    if (atomicAdd(sc + 1, 1u) == gridDim.x - 1) {
      sc[0] = 0;
      sc[1] = 0;
      __threadfence();
    }
  }
  if (kPair) cluster_sync_all();
  if (warp == 2) {
    tcgen05_fence_after();
    if (kPair) tmem_dealloc_pair(tmem_base, kAccBufs * kBN);
    else tmem_dealloc(tmem_base, kAccBufs * kBN);
  }
}

// Waits (bounded) until counters reach their targets: the consumer side of the
// TileGroup protocol when it runs as its own launch.  counter i = (src, g) with
// src-major layout; the target of group g is per_epoch[g] * epoch (counters only
// grow, one per_epoch[g] per launch); entries of `skip_src` are ignored.
__global__ void wait_groups_kernel(const uint32_t* sig, int sig_stride, int n_src, int n_groups,
                                   const uint32_t* per_epoch, uint32_t epoch, int skip_src,
                                   uint32_t* status, uint64_t budget_ns, int rank) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(budget_ns, &abort_word);
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_src * n_groups;
       i += gridDim.x * blockDim.x) {
    const int src = i / n_groups, g = i - src * n_groups;
    if (src == skip_src) continue;
    uint32_t seen = 0;
    const uint32_t target = per_epoch[g] * epoch;
    if (!tile_wait_ge(sig + src * sig_stride + g, target, wb, &seen)) {
      report_status(status, kStatusTimeoutSignal, 50, target, seen, rank, i);
      abort_word = 1;
      return;
    }
  }
}

static cudaError_t launch_fused_gemm_attrs_once() {
  static bool attr_set[64] = {};
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 64 && !attr_set[dev]) {
    e = cudaFuncSetAttribute(fused_gemm_sm100_kernel<false, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(fused_gemm_sm100_kernel<true, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(fused_gemm_sm100_kernel<true, true>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return e;
    attr_set[dev] = true;
  }
  return cudaSuccess;
}

cudaError_t launch_fused_gemm(const FusedGemmParams& p, int grid, cudaStream_t stream) {
  cudaError_t e = launch_fused_gemm_attrs_once();
  if (e != cudaSuccess) return e;
  fused_gemm_sm100_kernel<false, false><<<grid, kThreads, kSmemTotal, stream>>>(p);
  return cudaGetLastError();
}

// The CTA-pair form: clusters of two CTAs, `grid` even, always the rank's whole tile order.
cudaError_t launch_fused_gemm_pair(const FusedGemmParams& p, int grid, cudaStream_t stream,
                                   bool bounce) {
  cudaError_t e = launch_fused_gemm_attrs_once();
  if (e != cudaSuccess) return e;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(grid & ~1), 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kSmemTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (bounce) return cudaLaunchKernelEx(&cfg, fused_gemm_sm100_kernel<true, true>, p);
  return cudaLaunchKernelEx(&cfg, fused_gemm_sm100_kernel<true, false>, p);
}

// Forces the module that holds these kernels onto the current device (see tccl_preload_kernels).
cudaError_t preload_gemm_kernels() {
  cudaFuncAttributes a;
  cudaError_t e = cudaFuncGetAttributes(&a, fused_gemm_sm100_kernel<false, false>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, fused_gemm_sm100_kernel<true, false>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, fused_gemm_sm100_kernel<true, true>);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, wait_groups_kernel);
  if (e == cudaSuccess) e = launch_fused_gemm_attrs_once();
  return e;
}

cudaError_t launch_wait_groups(const uint32_t* sig, int sig_stride, int n_src, int n_groups,
                               const uint32_t* per_epoch, uint32_t epoch, int skip_src,
                               uint32_t* status, uint64_t budget_ns, int rank,
                               cudaStream_t stream) {
  int total = n_src * n_groups;
  int threads = 128;
  int blocks = (total + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  wait_groups_kernel<<<blocks, threads, 0, stream>>>(sig, sig_stride, n_src, n_groups, per_epoch,
                                                     epoch, skip_src, status, budget_ns, rank);
  return cudaGetLastError();
}

}  // namespace tileccl
