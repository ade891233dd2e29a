// Parameter block and constants shared by the fused tcgen05 GEMM kernel family
// (kernels/gemm_sm100.cu) and its host-side plan builder (gemm_plan.cc).
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace tileccl {

// CTA tile and pipeline shape.
static constexpr int kBM = 128;       // rows of C per tile (= UMMA M, one TMEM lane per row)
static constexpr int kBN = 256;       // columns of C per tile (= UMMA N, fp32 TMEM columns)
static constexpr int kBK = 64;        // K elements per stage (64 x 2 B = one 128-byte swizzle row)
static constexpr int kUmmaK = 16;     // K per tcgen05.mma for 16-bit inputs
static constexpr int kStages = 4;     // TMA -> MMA ring depth
static constexpr int kAccBufs = 2;    // TMEM accumulator double buffer (2 x 256 columns)
static constexpr int kEpiWarps = 4;   // epilogue warps (one per 32-lane TMEM quarter)
static constexpr int kThreads = 256;  // warp 0 TMA, 1 MMA, 2 TMEM alloc, 3 waiter, 4-7 epilogue
static constexpr int kChunkN = 64;    // epilogue column chunk (64 x 2 B = 128 B)
static constexpr int kSlabM = 32;     // rows per epilogue warp

static constexpr int kStageABytes = kBM * kBK * 2;
static constexpr int kStageBBytes = kBN * kBK * 2;
static constexpr int kStageBytes = kStageABytes + kStageBBytes;
static constexpr int kEpiBufBytes = kSlabM * kChunkN * 2;  // 4 KiB per (warp, buffer)
static constexpr int kEpiBufs = 2;
static constexpr int kSmemPipe = kStages * kStageBytes;
static constexpr int kSmemEpi = kEpiWarps * kEpiBufs * kEpiBufBytes;
static constexpr int kSmemCtl = 512;
static constexpr int kSmemTotal = kSmemPipe + kSmemEpi + kSmemCtl + 1024;  // + alignment slack

static constexpr int kMaxRanks = 8;
static constexpr int kStatPerCta = 4;      // counters per CTA row of the statistics table
static constexpr int kStatMaxCtas = 256;   // rows of the table (>= any grid of the kernel)

enum GemmMode : int {
  kModeGemm = 0,       // out[0] = A @ B
  kModePushAll = 1,    // every tile is stored to out[d] for all d (all-gather of the product)
  kModeReduceScatter = 2,  // tile goes to its owner's staging slot; owner tiles are reduced
  kModeAllScatter = 3,  // tile stored locally; tiles inside this rank's column slice go to all
};
enum PushMode : int {
  kPushStores = 0,  // peer copies with 16-byte st.global from the staged tile
  kPushTma = 1,     // peer copies with one TMA store per destination
  kPushMultimem = 2,  // one multimem.st per 16 bytes reaches every rank (needs NVLS)
};
enum TuningBits : int {
  // A TileGroup signal that follows a *completed* bulk store is sent as a relaxed add
  // instead of a release add.  Completion of a bulk group means the destination has
  // acknowledged the data, so an add issued afterwards cannot overtake it; a release add
  // would additionally wait for the younger bulk stores still in flight (measured: about
  // 6 us per tile and warp on NVLink 5 under load).
  kTuneRelaxedSignalAfterBulk = 1,
};
enum EpilogueOp : int {
  kEpiNone = 0,
  kEpiSiluGate = 1,  // out[:, j] = silu(acc[:, j]) * acc[:, 128 + j] per 256-column tile
};

struct alignas(64) FusedGemmParams {
  CUtensorMap tma_a;                  // A as [rows, K], box {64, 128}, 128B swizzle
  CUtensorMap tma_b;                  // B as [N, K] box {64, 256} or [K, N] box {64, 64}
  CUtensorMap tma_out[kMaxRanks];     // 3-D {cols, rows, slots}, box {64, 32, 1}
  // Reduce-scatter owners sum the peers' partial tiles on the tensor cores: a staged
  // partial tile P (128 x 256, 16-bit) enters the operand pipeline as a [K'=128, N=256]
  // B operand next to a 128 x 128 identity as A operand, so acc += I * P = P in fp32.
  CUtensorMap tma_stage;              // this rank's staging {cols, rows, slots}, box {64, 64, 1}
  CUtensorMap tma_ident;              // identity [128, 128], box {64, 128}
  // CTA-pair form of the kernel (gemm_sm100.cu, kPair): B with a box that covers 128 of a tile's 256 columns
  CUtensorMap tma_b_half;
  // raw views of the same destinations for the non-TMA push modes
  uint64_t out_ptr[kMaxRanks];
  uint64_t out_mc_ptr;                // multicast alias of the destination (push mode 2)
  int64_t out_ld_bytes;
  int64_t out_slot_bytes;             // bytes between staging slots (z coordinate)
  int32_t out_rows, out_cols;         // extent of one destination sub-matrix
  // problem
  int32_t mode, push_mode, epi_op, is_bf16, b_kmajor;
  int32_t rank, world_size;
  int32_t k_blocks;
  int32_t m_tiles_local, n_tiles_local;   // tiles of one owner's sub-problem
  int32_t owners;                          // 1, or world_size for reduce-scatter
  int32_t split_axis;                      // reduce-scatter: 0 = owners split rows, 1 = columns
  int32_t a_rows_per_owner, b_cols_per_owner;
  int32_t tile_begin, tile_end;            // half-open range of the rank's tile order to run
  int32_t rot_m_tiles;                     // plain GEMM: first m-tile to visit (others follow, wrapping)
  // TileGroup signalling (counters only ever grow)
  uint64_t sig_local;                 // this rank's counter array (uint32[sig_srcs][sig_stride])
  int64_t heap_stride;                // bytes between ranks' heaps: peer copy = sig_local + (d - rank) * stride
  int32_t sig_stride;                 // counters per source rank
  int32_t group_m_tiles;              // tile rows per TileGroup
  uint32_t epoch;                     // 1, 2, 3 ... per launch on this signal block
  int32_t wait_incoming;              // push-all: also wait for every peer's groups before exit
  // reduce-scatter staging on this rank: [2 parities][world_size][out_rows][out_cols]
  uint64_t stage_local;
  int32_t stage_parity;
  // A-operand gating (all-gather feeding this GEMM): uint32[world_size] arrival counters
  uint64_t a_gate;
  uint32_t a_gate_target;
  int32_t a_gate_rows_per_rank;
  // All-gather of the A operand done by warp 3 of every CTA while the GEMM runs:
  // this rank's `ag_bytes` at `ag_src` are copied to `ag_dst` in every peer's heap
  // (ag_dst is the local address of the destination region), then each CTA adds 1
  // to a_gate[rank] on every peer.  ag_bytes = 0 disables the role.
  uint64_t ag_src, ag_dst, ag_mc_dst;
  uint64_t ag_bytes;
  int32_t do_ag_push;
  // Entry handshake of the modes that write into buffers the peers also read (push-all,
  // all-scatter, all-gather of the A operand): uint32[world_size] on this rank, word s
  // counts the calls rank s has entered.  A rank adds 1 to word `rank` on every peer when
  // its kernel starts (its stream has then finished whatever read the previous call's
  // data) and stores into peer d only once word d here has reached `epoch`.  0 = off.
  uint64_t entry_local;
  int32_t announce_entry;             // this launch is the first of its call: announce it
  // column slice pushed by all-scatter
  int32_t scatter_col_begin, scatter_col_end;
  // Dynamic tile scheduling (launches that run the rank's whole tile order): uint32[2] in
  // device memory, {next position in the tile order, CTAs that have exited}; both are zero
  // between launches (the last CTA to exit resets them).  0 = static round-robin.
  uint64_t sched_counter;
  // diagnostics
  // optional uint64[kStatMaxCtas][kStatPerCta] table; CTA b of every launch adds its sums to
  // row b (the host adds up the rows and clears them): [0] bytes stored into peers' memory
  // [1] TileGroup signals sent  [2] SM cycles spent waiting for peers (TileGroup / gate
  // counters, summed over waiting threads)  [3] tiles computed
  uint64_t stats;
  uint64_t status;                    // uint32[kStatusWords]
  uint64_t wait_budget_ns;
  // optional uint64[trace_tile_slots][4 epilogue warps][4] (accumulator ready / stores
  // issued / older stores complete / signalled) followed by uint64[CTAs][8] (kernel entry /
  // roles start / incoming TileGroups seen / final CTA barrier passed / epilogue warp 0..3
  // done); a tile slot is a 128-row tile, in the CTA-pair form slot 2 * pair-tile + CTA
  uint64_t trace;
  int32_t trace_tile_slots;
  int32_t tuning;                     // TuningBits
  int32_t rs_own_lag;                 // TileOrderShape::own_lag
};

}  // namespace tileccl
