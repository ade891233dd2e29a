// C ABI of libtileccl_b200.so.  Python binds it with ctypes
// (tileccl_b200/_native.py); any other host language can do the same.
// Every function returns 0 on success and a non-zero code on failure, in which
// case tccl_last_error() describes what went wrong (thread-local string).
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCCL_MAX_RANKS 8

const char* tccl_last_error(void);
const char* tccl_version(void);
// Loads every kernel of the library onto the current device (call once per device, before
// kernels that wait on other ranks are in flight).
int tccl_preload_kernels(void);

// --------------------------------------------------------------------------
// Device / topology query (csrc/runtime/device.cc)
// --------------------------------------------------------------------------
typedef struct TcclDeviceProps {
  char name[128];
  int32_t ordinal;
  int32_t cc_major, cc_minor;
  int32_t sm_count;
  int32_t warp_size;
  int32_t max_smem_per_block_optin;
  int32_t l2_bytes;
  int32_t clock_khz, mem_clock_khz, mem_bus_bits;
  int32_t vmm_supported;
  int32_t posix_fd_handles;
  int32_t fabric_handles;
  int32_t multicast_supported;
  int64_t total_mem;
} TcclDeviceProps;

int tccl_device_count(int32_t* count);
int tccl_device_props(int32_t ordinal, TcclDeviceProps* out);
// access[i * n + j] = 1 when device i can map device j's memory; atomics likewise.
int tccl_peer_matrix(int32_t n, int32_t* access, int32_t* native_atomics);

// --------------------------------------------------------------------------
// Symmetric heap over cuMem VMM (csrc/runtime/symm_heap.cc)
// --------------------------------------------------------------------------
typedef struct TcclHeapInfo {
  uint64_t window_base;   // address of rank 0's heap in this process
  uint64_t stride;        // bytes between ranks (granularity-rounded heap size)
  uint64_t mc_base;       // multicast alias of this rank's heap offsets, 0 = none
  uint64_t requested_size;
  uint64_t granularity;
  int32_t rank, world_size;
  int32_t device;
  int32_t mode;           // 0 local_only, 1 single_process, 2 multiprocess
  int32_t transport;      // 0 none, 1 vmm_single_process, 2 vmm_fd, 3 vmm_fabric
  int32_t nvls_bound;
} TcclHeapInfo;

// One process maps every rank (rank r lives on device devices[r]); returns one
// handle per rank that share the same window.
int tccl_heap_create_local(int32_t world_size, uint64_t size, const int32_t* devices,
                           int32_t want_nvls, void** handles_out);
// One process per rank.  Collective: every rank calls it with the same job id;
// allocation handles travel as file descriptors over abstract Unix sockets.
int tccl_heap_create_multiprocess(int32_t rank, int32_t world_size, uint64_t size, int32_t device,
                                  const char* job_id, int32_t want_nvls, int32_t timeout_ms,
                                  void** handle_out);
int tccl_heap_info(void* handle, TcclHeapInfo* out);
int tccl_heap_destroy(void* handle);

// 256-byte aligned bump allocation inside the heap (never freed individually).
int tccl_heap_alloc(void* handle, uint64_t bytes, uint64_t* offset_out);
int tccl_heap_reset(void* handle);
int tccl_heap_bytes_allocated(void* handle, uint64_t* out);

// Rendezvous layer on its own (host only): all-gathers one (payload, fd) per rank
// over abstract Unix sockets.  fds_out[r] is a descriptor valid in the caller.
int tccl_bootstrap_allgather(int32_t rank, int32_t world_size, const char* job_id,
                             int32_t timeout_ms, uint64_t payload, int32_t fd,
                             uint64_t* payloads_out, int32_t* fds_out);

// --------------------------------------------------------------------------
// Fused tcgen05 GEMM family (csrc/kernels/gemm_sm100.cu)
// --------------------------------------------------------------------------
typedef struct TcclGemmDesc {
  int32_t mode;        // 0 gemm, 1 push-all, 2 reduce-scatter, 3 all-scatter
  int32_t dtype;       // 0 fp16, 1 bf16 (inputs and outputs; accumulation is fp32)
  int32_t b_kmajor;    // 0: B is [K, N] row-major; 1: B is [N, K] row-major
  int32_t epi_op;      // 0 none, 1 SiLU-gate
  int32_t push_mode;   // 0 st.global, 1 TMA store, 2 multimem.st
  int32_t rank, world_size;
  int32_t split_axis;  // reduce-scatter: 0 = owners split rows of C, 1 = columns
  int64_t a_rows;      // rows of A that may be read
  int64_t b_cols;      // columns of B that may be read
  int64_t k;
  uint64_t a_ptr; int64_t lda;   // leading dimensions in elements
  uint64_t b_ptr; int64_t ldb;
  int64_t sub_m, sub_n;          // accumulator extent of one owner's sub-problem
  uint64_t out_ptr[TCCL_MAX_RANKS];
  uint64_t out_mc_ptr;
  int64_t ldo;                   // elements
  int64_t out_rows, out_cols;    // extent of one destination sub-matrix
  int64_t out_slot_elems;        // elements between slots (reduce-scatter staging), else 0
  int32_t out_slots;             // >= 1
  int32_t group_m_tiles;
  uint64_t sig_local; int64_t heap_stride; int32_t sig_stride;
  int32_t rot_m_tiles;
  uint64_t stage_local;
  uint64_t a_gate; int32_t a_gate_rows_per_rank;
  // all-gather of the A operand pushed by the kernel itself (0 bytes = off)
  uint64_t ag_src, ag_dst, ag_mc_dst, ag_bytes;
  int32_t scatter_col_begin, scatter_col_end;
  int32_t grid;                  // 0 = one CTA per SM
  uint64_t stats;                // uint64[256][4] in device memory, may be 0: CTA b of every launch adds its
                                 // counters to row b (bytes stored to peers, signals sent, SM cycles waited
                                 // for peers, tiles)
  uint64_t status;               // uint32[8] in device memory, may be 0
  uint64_t trace;                // uint64[TcclGemmPlanInfo::trace_words] in device memory, may be 0: 4 stamps per
                                 // epilogue warp and 128-row tile, then 4 stamps per CTA
  uint64_t wait_budget_ns;       // 0 = default (2 s)
  int32_t tuning;                // bit 0: TileGroup signals after a completed bulk store are relaxed adds
  int32_t rs_own_lag;            // reduce-scatter: rounds by which the own (reducing) tile rows trail; 0 = all last
  uint64_t ident_ptr;            // reduce-scatter: 128 x 128 identity matrix of the operand dtype (row-major)
  int32_t disable_cta_pairs;     // 1: whole-order launches also run the one-CTA form
  int32_t comm_ctas;             // reserved (0)
  int32_t dynamic_tiles;         // 1: whole-order launches hand tiles to CTAs from a global counter
  int32_t reserved0;
  uint64_t entry_local;          // uint32[world_size] "calls entered" counters of this rank on the heap
                                 // (entry handshake of the modes that store into peers' buffers), 0 = off
} TcclGemmDesc;

typedef struct TcclGemmPlanInfo {
  int32_t grid;
  int32_t tiles_total;       // tiles in this rank's order
  int32_t tiles_per_owner;
  int32_t m_tiles_local, n_tiles_local;
  int32_t groups;            // TileGroups per owner sub-problem
  int32_t k_blocks;
  int32_t smem_bytes;
  int32_t push_grid;         // CTAs of a launch that performs the all-gather push
  int32_t pair_kernel;       // 1: whole-order launches run the CTA-pair form
  int32_t pair_grid;         // CTAs of such a launch
  int64_t trace_words;       // uint64 words a trace buffer (TcclGemmDesc::trace) must hold
} TcclGemmPlanInfo;

int tccl_gemm_plan_create(const TcclGemmDesc* desc, void** plan_out);
int tccl_gemm_plan_info(void* plan, TcclGemmPlanInfo* out);
// epoch: 1, 2, 3 ... per launch on the plan's signal block (ignored by mode 0).
// tile_end < 0 runs to the last tile.  flags: bit 0 = also wait for every peer's
// TileGroups before the kernel exits (push-all), bit 1 = perform the all-gather push
// of the A operand (an empty tile range is then allowed: push only), bit 3 = this is the
// first launch of its call: tell the peers that this rank has entered it (entry handshake).
int tccl_gemm_plan_launch(void* plan, uint32_t epoch, uint32_t a_gate_target, int32_t tile_begin,
                          int32_t tile_end, int32_t flags, uint64_t stream);
// The same launch while the A operand is still arriving from pinned host memory: for each
// run of tiles, the listed byte ranges are copied host -> device on `copy_stream`
// (one cudaMemcpyAsync per range), and the run is launched on `stream` as soon as its
// copies are done.  The copies start after everything queued on `stream` so far (earlier
// readers of A); with flags bit 2 they only follow this plan's previous streamed call (the
// caller promises that no other pending work on `stream` touches A), so the copy of one
// problem overlaps the kernels of the previous one.  Bit 0 applies to the last run, bit 1 to
// the first.  With `copy_stream2` != 0 the runs' copies alternate between the two copy
// streams, so that the set-up of one copy hides under the transfer of the other.
#define TCCL_STREAM_MAX_RANGES 64
typedef struct TcclStreamChunk {
  int32_t tile_begin, tile_end;
  int32_t n_ranges;
  int32_t reserved;
  uint64_t dst[TCCL_STREAM_MAX_RANGES];     // device addresses
  uint64_t src[TCCL_STREAM_MAX_RANGES];     // pinned host addresses
  uint64_t bytes[TCCL_STREAM_MAX_RANGES];
} TcclStreamChunk;
int tccl_gemm_plan_launch_streamed(void* plan, uint32_t epoch, uint32_t a_gate_target,
                                   int32_t flags, const TcclStreamChunk* chunks, int32_t n_chunks,
                                   uint64_t copy_stream, uint64_t copy_stream2, uint64_t stream);
int tccl_gemm_plan_destroy(void* plan);

// Consumer side of the TileGroup protocol as its own launch: waits until
// sig[src * sig_stride + g] >= per_epoch[g] * epoch for every src != skip_src.
int tccl_wait_groups(uint64_t sig, int32_t sig_stride, int32_t n_src, int32_t n_groups,
                     uint64_t per_epoch, uint32_t epoch, int32_t skip_src, uint64_t status,
                     uint64_t budget_ns, int32_t rank, uint64_t stream);

// --------------------------------------------------------------------------
// Tile collectives on heap buffers (csrc/kernels/collectives.cu)
// op: 0 all-gather, 1 reduce-scatter, 2 all-reduce (two-shot), 3 all-reduce (one-shot),
//     4 broadcast, 5 scatter.  dtype: 0 fp16, 1 bf16, 2 fp32, 3 raw bytes (copy ops only).
// phase_mask: bit 0 announce, bit 1 move data, bit 2 wait for completion (7 = whole call).
// staging / stage_slot (one-shot all-reduce): two parity halves, the second at
// staging + stage_slot (0: directly behind the first, at the message size rounded to 16).
// --------------------------------------------------------------------------
int tccl_collective_launch(int32_t op, int32_t dtype, int32_t rank, int32_t world_size,
                           int32_t root, int32_t use_multimem, int32_t phase_mask, int32_t elem_size,
                           uint32_t epoch,
                           uint64_t src, uint64_t dst, uint64_t staging, uint64_t stage_slot,
                           uint64_t counters,
                           uint64_t mc_base, uint64_t heap_base, int64_t heap_stride,
                           uint64_t bytes, int32_t grid, uint64_t status, uint64_t budget_ns,
                           uint64_t stream);

// Low-latency form of all-gather, broadcast, scatter (op 0, 4, 5), reduce-scatter (op 1) and
// one-shot all-reduce (op 3, in place: src == dst; `dtype` 0 fp16 / 1 bf16 / 2 fp32 for the
// two reductions, ignored by the copies) for messages of at most 1 MiB
// per (source, destination): payload and flag travel in the same 16-byte store.  `stage`:
// this rank's zeroed staging on the heap, 2 x slots x slot_bytes (slots = world_size for
// all-gather, reduce-scatter and all-reduce, else 1; slot_bytes >= 2 x bytes, at least 128 KiB);
// `counters`: 32 zeroed uint32 on the heap; both per collective kind, root and slot size.
// phase_mask: bit 0 send, bit 1 receive (3 = whole call).
int tccl_collective_ll_launch(int32_t op, int32_t dtype, int32_t rank, int32_t world_size,
                              int32_t root,
                              int32_t phase_mask, uint32_t epoch, uint64_t src, uint64_t dst,
                              uint64_t stage, uint64_t counters, int64_t heap_stride,
                              uint64_t bytes, uint64_t slot_bytes, int32_t grid, uint64_t status,
                              uint64_t budget_ns, uint64_t stream);

// Pipelined relay broadcast for large messages on 3..8 ranks: the root sends piece p of
// `buf` (pieces of `piece_bytes`, at most 16384 of them) once, to the non-root ranks in turn,
// with a flag; each of those forwards its pieces to the other non-root ranks.  `flags`:
// 16384 zeroed uint32 on the heap, `counters`: 32 zeroed uint32 on the heap, both per root.
// phase_mask: 1 announce, 2 root push, 8 relay forwarding, 4 final wait (15 = whole call).
// `bulk` != 0: bulk copies through shared memory, four pipelines per CTA (grid counts CTAs
// of 128 threads); 0: register copies by CTAs of 512 threads.
int tccl_broadcast_relay_launch(int32_t rank, int32_t world_size, int32_t root,
                                int32_t phase_mask, uint32_t epoch, uint64_t buf, uint64_t bytes,
                                uint64_t piece_bytes, uint64_t flags, uint64_t counters,
                                uint64_t heap_base, int64_t heap_stride, int32_t grid, int32_t bulk,
                                uint64_t status, uint64_t budget_ns, uint64_t stream);

// --------------------------------------------------------------------------
// Region push (csrc/kernels/push_region.cu): copies rows x row_bytes (pitch
// ld_bytes) of this rank's heap to the same place in every peer's heap, band by
// band; optionally waits for a local per-band counter (band_ready) first.
// --------------------------------------------------------------------------
int tccl_push_region(uint64_t region, uint64_t mc_region, int64_t ld_bytes, int32_t rows,
                     int32_t row_bytes, int32_t band_rows, int32_t rank, int32_t world_size,
                     int64_t heap_stride, uint64_t band_ready, uint32_t band_target_per_epoch,
                     uint64_t counters, uint32_t epoch, int32_t phase_mask, int32_t grid,
                     uint64_t status, uint64_t budget_ns, uint64_t stream);

// --------------------------------------------------------------------------
// TileGroup planner (csrc/plan/tile_group.cc, host only).  groups_out holds
// (row_start, row_end, tile_count) triples.
// --------------------------------------------------------------------------
int tccl_plan_tile_groups(int64_t M, int64_t N, int64_t tile_bytes, int64_t target_group_tiles,
                          int32_t max_groups, int32_t block_m, int32_t block_n, int32_t group_m,
                          int64_t tau_min_bytes, const int64_t* row_boundaries,
                          int32_t n_boundaries, int64_t* groups_out, int32_t capacity,
                          int32_t* n_groups_out);
int tccl_plan_group_table(int64_t M, int64_t N, const int64_t* groups, int32_t n_groups,
                          int32_t block_m, int32_t block_n, int32_t group_m, int32_t* table_out,
                          int64_t table_len);

// --------------------------------------------------------------------------
// CPU emulation of the multi-rank fused operators (csrc/cpu_emul/fake_device.cc):
// one thread per rank, fp32, same tile order and TileGroup signalling as the GPU
// kernels.  fault_kind: 0 none, 1 never signals, 2 signals every other tile only,
// 3 rank absent, 4 rank late by fault_delay_ms.  status_out: int32[6] =
// {code (0 ok, 2 = a wait timed out), where, rank, item, expected, observed}.
// --------------------------------------------------------------------------
int tccl_emul_gemm_allgather(int32_t world_size, int32_t M, int32_t N, int32_t K,
                             const float* A_all, const float* B_all, float* C_all,
                             int32_t block_m, int32_t block_n, int32_t group_m_tiles,
                             int32_t fault_rank, int32_t fault_kind, int32_t fault_delay_ms,
                             int32_t timeout_ms, int32_t* status_out);
int tccl_emul_gemm_reducescatter(int32_t world_size, int32_t M, int32_t N, int32_t K_total,
                                 const float* A_all, const float* B_all, float* C_all,
                                 int32_t block_m, int32_t block_n, int32_t group_m_tiles,
                                 int32_t fault_rank, int32_t fault_kind, int32_t fault_delay_ms,
                                 int32_t timeout_ms, int32_t* status_out);
int tccl_emul_gemm_reducescatter_ex(int32_t world_size, int32_t M, int32_t N, int32_t K_total,
                                    const float* A_all, const float* B_all, float* C_all,
                                    int32_t block_m, int32_t block_n, int32_t group_m_tiles,
                                    int32_t own_lag, int32_t signal_delay_tiles,
                                    int32_t flush_before_wait, int32_t fault_rank,
                                    int32_t fault_kind, int32_t fault_delay_ms, int32_t timeout_ms,
                                    int32_t* status_out);
// (owner, tile row, tile column) of every tile in one rank's visiting order.
int tccl_plan_tile_order(int32_t m_tiles_local, int32_t n_tiles_local, int32_t owners, int32_t rank,
                         int32_t world_size, int32_t rot_m_tiles, int32_t* out, int32_t capacity);
// Same, with the reduce-scatter own rows trailing the remote rounds by `own_lag` (0 = all last).
int tccl_plan_tile_order_ex(int32_t m_tiles_local, int32_t n_tiles_local, int32_t owners,
                            int32_t rank, int32_t world_size, int32_t rot_m_tiles, int32_t own_lag,
                            int32_t* out, int32_t capacity);

// --------------------------------------------------------------------------
// Device-primitive test harness (csrc/kernels/prim_test.cu): one launch acts as
// `rank` and applies one primitive.  op codes: 0 put, 1 get, 2 remote_store,
// 3 remote_load, 4 signal, 5 wait, 6 poll, 7 signal_add, 8 wait_ge, 9 atomic
// (sub_op 0 add, 1 cas, 2 xchg, 3 min, 4 max, 5 and, 6 or, 7 xor), 10 barrier,
// 11 credit (sub_op 0 acquire, 1 release), 12 try_wait, 13 translate,
// 14 put_mc, 15 get_reduce.  `result` is uint32[4] in device memory.
// --------------------------------------------------------------------------
// Grid-wide point-to-point copy with the tile_put / tile_get accessors: direction 0 puts the
// local `a` into `peer`'s `b`, direction 1 gets `peer`'s `a` into the local `b` (symmetric
// addresses are given as addresses in the caller's heap).
int tccl_p2p_copy(int32_t direction, int32_t rank, int32_t world_size, int32_t peer,
                  uint64_t window_base, uint64_t stride, uint64_t a, uint64_t b, uint64_t bytes,
                  int32_t grid, uint64_t stream);
int tccl_prim_test(int32_t op, int32_t sub_op, int32_t rank, int32_t world_size, int32_t peer,
                   uint64_t window_base, uint64_t stride, uint64_t mc_base, uint64_t a, uint64_t b,
                   uint64_t n, uint32_t value, uint32_t value2, uint64_t result, uint64_t budget_ns,
                   uint64_t stream);

// --------------------------------------------------------------------------
// Debug build (-DTILECCL_DEBUG_CHECKS, libtileccl_b200_debug.so): the record of bounds
// violations of the current device (tileccl::DebugRecord in device/symm_ptr.cuh, 40 bytes:
// count, code, rank, from_rank, to_rank, enabled, addr, bytes), one per translation unit
// that uses the device primitives.  `enabled` is 0 in a release build.  `clear` != 0
// zeroes the record after reading.  Call after synchronising the streams of interest.
// --------------------------------------------------------------------------
int tccl_debug_read_primitives(void* out_record, int32_t clear);   // prim_test.cu kernels
int tccl_debug_read_collectives(void* out_record, int32_t clear);  // collectives.cu kernels

#ifdef __cplusplus
}
#endif
