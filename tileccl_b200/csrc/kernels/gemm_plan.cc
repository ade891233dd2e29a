// Host side of the fused GEMM family: validates a TcclGemmDesc, encodes the TMA
// tensor maps once, and keeps the resulting parameter block so that repeated
// launches (the normal case: one plan per layer, many steps) cost one kernel
// launch and no driver calls.
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <memory>
#include <vector>

#include "../api.h"
#include "../runtime/errors.h"
#include "gemm_sm100.cuh"

namespace tileccl {
cudaError_t launch_fused_gemm(const FusedGemmParams& p, int grid, cudaStream_t stream);
cudaError_t launch_fused_gemm_pair(const FusedGemmParams& p, int grid, cudaStream_t stream,
                                   bool bounce);
cudaError_t preload_gemm_kernels();
cudaError_t preload_collective_kernels();
cudaError_t preload_push_kernels();
cudaError_t preload_prim_kernels();
cudaError_t launch_wait_groups(const uint32_t* sig, int sig_stride, int n_src, int n_groups,
                               const uint32_t* per_epoch, uint32_t epoch, int skip_src,
                               uint32_t* status, uint64_t budget_ns, int rank,
                               cudaStream_t stream);

namespace {

struct GemmPlan {
  FusedGemmParams params;
  TcclGemmPlanInfo info;
  bool pair_kernel = false;   // whole-order launches run on CTA pairs
  int pair_grid = 0, pair_push_grid = 0;
  std::vector<cudaEvent_t> events;   // streamed launches: one per run of tiles, + 1
  cudaEvent_t done_event = nullptr;  // end of the last streamed call on its launch stream
  bool streamed_before = false;
  // Dynamic tile scheduler: {next position, exited CTAs}.  Allocated at the first
  // whole-order launch, on the device that launch runs on (a plan may be built while another
  // device is current, e.g. one process driving several GPUs).
  bool want_sched = false;
  uint32_t* sched = nullptr;
  int sched_device = -1;
  ~GemmPlan() {
    if (sched != nullptr) cudaFree(sched);
    for (cudaEvent_t e : events) cudaEventDestroy(e);
    if (done_event != nullptr) cudaEventDestroy(done_event);
  }
};

// 16-bit row-major matrix [rows, cols] (+ optional slot dimension) -> tensor map
// with a {box_cols, box_rows(, 1)} box and 128-byte swizzle.
int encode_map(CUtensorMap* map, bool bf16, uint64_t base, uint64_t cols, uint64_t rows,
               uint64_t ld_bytes, uint32_t box_cols, uint32_t box_rows, uint64_t slots,
               uint64_t slot_bytes, const char* what) {
  const DriverApi& d = driver();
  TCCL_CHECK_ARG(base % 16 == 0, what << ": base address must be 16-byte aligned");
  TCCL_CHECK_ARG(ld_bytes % 16 == 0, what << ": row pitch must be a multiple of 16 bytes");
  CUtensorMapDataType dt = bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (slots == 0) {
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {ld_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t es[2] = {1, 1};
    CUresult r = d.cuTensorMapEncodeTiled(map, dt, 2, reinterpret_cast<void*>(base), dims, strides,
                                          box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          CU_TENSOR_MAP_SWIZZLE_128B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return fail(kErrCuda, std::string("cuTensorMapEncodeTiled(") + what + "): " +
                                driver_error_string(r));
  } else {
    TCCL_CHECK_ARG(slot_bytes % 16 == 0, what << ": slot pitch must be a multiple of 16 bytes");
    cuuint64_t dims[3] = {cols, rows, slots};
    cuuint64_t strides[2] = {ld_bytes, slot_bytes};
    cuuint32_t box[3] = {box_cols, box_rows, 1};
    cuuint32_t es[3] = {1, 1, 1};
    CUresult r = d.cuTensorMapEncodeTiled(map, dt, 3, reinterpret_cast<void*>(base), dims, strides,
                                          box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                          CU_TENSOR_MAP_SWIZZLE_128B,
                                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS)
      return fail(kErrCuda, std::string("cuTensorMapEncodeTiled(") + what + "): " +
                                driver_error_string(r));
  }
  return kOk;
}

int build_plan(const TcclGemmDesc& d, GemmPlan* plan) {
  TCCL_REQUIRE_DRIVER();
  TCCL_CHECK_ARG(d.mode >= 0 && d.mode <= 3, "mode must be 0..3");
  TCCL_CHECK_ARG(d.dtype == 0 || d.dtype == 1, "dtype must be 0 (fp16) or 1 (bf16)");
  TCCL_CHECK_ARG(d.world_size >= 1 && d.world_size <= kMaxRanks, "world_size must be 1..8");
  TCCL_CHECK_ARG(d.rank >= 0 && d.rank < d.world_size, "rank out of range");
  TCCL_CHECK_ARG(d.k > 0 && d.a_rows > 0 && d.b_cols > 0, "empty problem");
  TCCL_CHECK_ARG(d.sub_m > 0 && d.sub_n > 0, "empty sub-problem");
  TCCL_CHECK_ARG(d.k % 8 == 0, "K must be a multiple of 8 (16-byte TMA rows)");
  TCCL_CHECK_ARG(d.lda % 8 == 0 && d.ldb % 8 == 0 && d.ldo % 8 == 0,
                 "leading dimensions must be multiples of 8 elements");
  TCCL_CHECK_ARG(d.out_cols % 8 == 0, "output columns must be a multiple of 8");
  TCCL_CHECK_ARG(d.group_m_tiles >= 1, "group_m_tiles must be >= 1");
  TCCL_CHECK_ARG(d.push_mode >= 0 && d.push_mode <= 2, "push_mode must be 0..2");
  if (d.epi_op == kEpiSiluGate)
    TCCL_CHECK_ARG(d.sub_n % kBN == 0, "SiLU-gate epilogue needs sub_n to be a multiple of 256");
  if (d.push_mode == kPushMultimem)
    TCCL_CHECK_ARG(d.out_mc_ptr != 0, "push_mode 2 needs a multicast destination");

  FusedGemmParams& p = plan->params;
  std::memset(&p, 0, sizeof(p));
  const bool bf16 = d.dtype == 1;

  int rc = encode_map(&p.tma_a, bf16, d.a_ptr, d.k, d.a_rows, d.lda * 2, kBK, kBM, 0, 0, "A");
  if (rc) return rc;
  if (d.b_kmajor)
    rc = encode_map(&p.tma_b, bf16, d.b_ptr, d.k, d.b_cols, d.ldb * 2, kBK, kBN, 0, 0, "B[N,K]");
  else
    rc = encode_map(&p.tma_b, bf16, d.b_ptr, d.b_cols, d.k, d.ldb * 2, 64, kBK, 0, 0, "B[K,N]");
  if (rc) return rc;

  const int n_dest = d.mode == kModeGemm ? 1 : d.world_size;
  const uint64_t slots = d.out_slots > 0 ? d.out_slots : 1;
  const uint64_t slot_bytes =
      d.out_slot_elems > 0 ? d.out_slot_elems * 2 : static_cast<uint64_t>(d.out_rows) * d.ldo * 2;
  for (int i = 0; i < n_dest; ++i) {
    TCCL_CHECK_ARG(d.out_ptr[i] != 0, "missing destination " << i);
    // In reduce-scatter mode only the peers' entries are staging (many slots);
    // this rank's own entry is the final C shard (one slot).
    const bool is_staging = d.mode == kModeReduceScatter && i != d.rank;
    rc = encode_map(&p.tma_out[i], bf16, d.out_ptr[i], d.out_cols, d.out_rows, d.ldo * 2, kChunkN,
                    kSlabM, is_staging ? slots : 1, is_staging ? slot_bytes
                                                               : static_cast<uint64_t>(d.out_rows) * d.ldo * 2,
                    "out");
    if (rc) return rc;
    p.out_ptr[i] = d.out_ptr[i];
  }
  // B for the CTA-pair kernel: each CTA of a pair loads 128 of the tile's 256 columns.
  if (d.b_kmajor)
    rc = encode_map(&p.tma_b_half, bf16, d.b_ptr, d.k, d.b_cols, d.ldb * 2, kBK, kBN / 2, 0, 0,
                    "B[N,K] half");
  else
    rc = encode_map(&p.tma_b_half, bf16, d.b_ptr, d.b_cols, d.k, d.ldb * 2, 64, kBK, 0, 0,
                    "B[K,N] half");
  if (rc) return rc;
  if (d.mode == kModeReduceScatter && d.world_size > 1) {
    TCCL_CHECK_ARG(d.stage_local != 0, "reduce-scatter needs this rank's staging area");
    TCCL_CHECK_ARG(d.ident_ptr != 0, "reduce-scatter needs the 128 x 128 identity operand");
    rc = encode_map(&p.tma_stage, bf16, d.stage_local, d.out_cols, d.out_rows, d.ldo * 2, 64, kBK,
                    slots, slot_bytes, "staging");
    if (rc) return rc;
    rc = encode_map(&p.tma_ident, bf16, d.ident_ptr, kBM, kBM, kBM * 2, kBK, kBM, 0, 0, "identity");
    if (rc) return rc;
  }
  p.out_mc_ptr = d.out_mc_ptr;
  p.out_ld_bytes = d.ldo * 2;
  p.out_slot_bytes = static_cast<int64_t>(slot_bytes);
  p.out_rows = static_cast<int32_t>(d.out_rows);
  p.out_cols = static_cast<int32_t>(d.out_cols);

  p.mode = d.mode;
  p.push_mode = d.push_mode;
  p.epi_op = d.epi_op;
  p.is_bf16 = bf16 ? 1 : 0;
  p.b_kmajor = d.b_kmajor ? 1 : 0;
  p.rank = d.rank;
  p.world_size = d.world_size;
  p.k_blocks = static_cast<int32_t>((d.k + kBK - 1) / kBK);
  p.m_tiles_local = static_cast<int32_t>((d.sub_m + kBM - 1) / kBM);
  p.n_tiles_local = static_cast<int32_t>((d.sub_n + kBN - 1) / kBN);
  p.owners = d.mode == kModeReduceScatter ? d.world_size : 1;
  p.split_axis = d.split_axis;
  p.a_rows_per_owner = static_cast<int32_t>(d.sub_m);
  p.b_cols_per_owner = static_cast<int32_t>(d.sub_n);
  p.rot_m_tiles = d.rot_m_tiles;
  TCCL_CHECK_ARG(p.rot_m_tiles >= 0 && p.rot_m_tiles < p.m_tiles_local, "rot_m_tiles out of range");
  p.sig_local = d.sig_local;
  p.heap_stride = d.heap_stride;
  p.sig_stride = d.sig_stride;
  p.group_m_tiles = d.group_m_tiles;
  p.stage_local = d.stage_local;
  p.a_gate = d.a_gate;
  p.a_gate_rows_per_rank = d.a_gate_rows_per_rank > 0 ? d.a_gate_rows_per_rank : 1;
  p.ag_src = d.ag_src;
  p.ag_dst = d.ag_dst;
  p.ag_mc_dst = d.ag_mc_dst;
  p.ag_bytes = d.ag_bytes;
  if (d.ag_bytes != 0) {
    TCCL_CHECK_ARG(d.ag_bytes % 16 == 0 && d.ag_src % 16 == 0 && d.ag_dst % 16 == 0,
                   "all-gather push needs 16-byte aligned buffers and size");
    TCCL_CHECK_ARG(d.a_gate != 0 && d.heap_stride != 0, "all-gather push needs gate counters");
  }
  p.entry_local = d.entry_local;
  if (d.entry_local != 0)
    TCCL_CHECK_ARG(d.heap_stride != 0 && d.entry_local % 4 == 0,
                   "the entry handshake needs the heap stride and aligned counters");
  p.scatter_col_begin = d.scatter_col_begin;
  p.scatter_col_end = d.scatter_col_end;
  p.status = d.status;
  p.stats = d.stats;
  p.trace = d.trace;
  p.tuning = d.tuning;
  TCCL_CHECK_ARG(d.rs_own_lag >= 0, "rs_own_lag must be >= 0");
  p.rs_own_lag = d.mode == kModeReduceScatter ? d.rs_own_lag : 0;
  p.wait_budget_ns = d.wait_budget_ns ? d.wait_budget_ns : 2000000000ull;

  const int groups = (p.m_tiles_local + p.group_m_tiles - 1) / p.group_m_tiles;
  if (d.world_size > 1 && d.mode != kModeGemm) {
    TCCL_CHECK_ARG(d.sig_local != 0, "multi-rank modes need a signal block");
    TCCL_CHECK_ARG(groups <= d.sig_stride, "signal block has fewer counters than TileGroups");
    if (d.mode == kModeReduceScatter)
      TCCL_CHECK_ARG(d.stage_local != 0, "reduce-scatter needs a staging buffer");
  }
  if (d.mode == kModeAllScatter)
    TCCL_CHECK_ARG(d.scatter_col_begin % kChunkN == 0,
                   "all-scatter column slice must start on a multiple of 64");

  int grid = d.grid;
  if (grid <= 0) {
    int dev = 0, sms = 0;
    TCCL_CHECK_CUDA(cudaGetDevice(&dev));
    TCCL_CHECK_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    grid = sms;
  }
  TcclGemmPlanInfo& info = plan->info;
  info.tiles_per_owner = p.m_tiles_local * p.n_tiles_local;
  info.tiles_total = info.tiles_per_owner * p.owners;
  info.grid = grid < info.tiles_total ? grid : info.tiles_total;
  info.push_grid = grid;
  info.m_tiles_local = p.m_tiles_local;
  info.n_tiles_local = p.n_tiles_local;
  info.groups = groups;
  info.k_blocks = p.k_blocks;
  info.smem_bytes = kSmemTotal;

  // Launches that run the rank's whole tile order use CTA pairs (256 x 256 per pair, see
  // gemm_sm100.cu); tile-range launches (emulated ranks, host-streamed operand) and
  // explicit grids stay on the one-CTA form.
  const bool allowed = d.disable_cta_pairs == 0;
  plan->pair_kernel = allowed && d.rot_m_tiles % 2 == 0 && d.grid <= 0 && grid >= 2 &&
                      grid % 2 == 0;
  if (plan->pair_kernel) {
    const int pair_tiles = ((p.m_tiles_local + 1) / 2) * p.n_tiles_local * p.owners;
    const int pairs = grid / 2 < pair_tiles ? grid / 2 : pair_tiles;
    plan->pair_grid = 2 * pairs;
    plan->pair_push_grid = grid & ~1;
  }
  // Dynamic tile scheduling evens out unequal shares of the link; a single rank has no link
  // and keeps the fixed order (best L2 reuse, no scheduling traffic).
  plan->want_sched = d.dynamic_tiles != 0 && d.world_size > 1;
  info.pair_kernel = plan->pair_kernel ? 1 : 0;
  info.pair_grid = plan->pair_grid;
  // uint64 words a trace buffer must hold: tile slots of the larger form + per-CTA stamps
  {
    const int64_t slots_one = info.tiles_total;
    const int64_t slots_pair =
        2ll * ((p.m_tiles_local + 1) / 2) * p.n_tiles_local * p.owners;
    info.trace_words = (slots_one > slots_pair ? slots_one : slots_pair) * 16 + 8ll * grid;
  }
  return kOk;
}

}  // namespace
}  // namespace tileccl

using namespace tileccl;

extern "C" int tccl_gemm_plan_create(const TcclGemmDesc* desc, void** plan_out) {
  TCCL_CHECK_ARG(desc != nullptr && plan_out != nullptr, "null argument");
  std::unique_ptr<GemmPlan> plan(new GemmPlan());
  int rc = build_plan(*desc, plan.get());
  if (rc) return rc;
  *plan_out = plan.release();
  return kOk;
}

extern "C" int tccl_gemm_plan_info(void* plan, TcclGemmPlanInfo* out) {
  TCCL_CHECK_ARG(plan != nullptr && out != nullptr, "null argument");
  *out = static_cast<GemmPlan*>(plan)->info;
  return kOk;
}

extern "C" int tccl_gemm_plan_launch(void* plan_, uint32_t epoch, uint32_t a_gate_target,
                                     int32_t tile_begin, int32_t tile_end, int32_t flags,
                                     uint64_t stream) {
  TCCL_CHECK_ARG(plan_ != nullptr, "null plan");
  GemmPlan* plan = static_cast<GemmPlan*>(plan_);
  FusedGemmParams p = plan->params;
  const int total = plan->info.tiles_total;
  if (tile_end < 0 || tile_end > total) tile_end = total;
  TCCL_CHECK_ARG(tile_begin >= 0 && tile_begin <= tile_end, "bad tile range");
  const bool ag_push = (flags & 2) != 0 && plan->params.ag_bytes != 0;
  if (tile_begin == tile_end && !ag_push) return kOk;
  p.tile_begin = tile_begin;
  p.tile_end = tile_end;
  p.epoch = epoch;
  p.stage_parity = static_cast<int32_t>(epoch & 1u);
  p.a_gate_target = a_gate_target;
  p.wait_incoming = (flags & 1) ? 1 : 0;
  p.do_ag_push = ag_push ? 1 : 0;
  p.announce_entry = (flags & 8) ? 1 : 0;
  // Whole-order launches hand tiles out dynamically; tile-range launches (several launches
  // share one order) keep the fixed round-robin assignment.
  p.sched_counter = 0;
  if (plan->want_sched && tile_begin == 0 && tile_end == total && total > 0) {
    int dev = -1;
    TCCL_CHECK_CUDA(cudaGetDevice(&dev));
    if (plan->sched == nullptr) {
      // Two counters that every whole-order launch finds, and leaves, at zero.
      TCCL_CHECK_CUDA(cudaMalloc(reinterpret_cast<void**>(&plan->sched), 2 * sizeof(uint32_t)));
      TCCL_CHECK_CUDA(cudaMemset(plan->sched, 0, 2 * sizeof(uint32_t)));
      plan->sched_device = dev;
    }
    TCCL_CHECK_ARG(dev == plan->sched_device,
                   "this plan was first launched on device " << plan->sched_device
                                                             << " and cannot move to device " << dev);
    p.sched_counter = reinterpret_cast<uint64_t>(plan->sched);
  }
  int grid = plan->info.grid;
  if (ag_push) {
    // Every CTA contributes one arrival to the peers' gate counters, so the grid of a
    // pushing launch is fixed (the consumers expect epoch * grid arrivals).
    grid = plan->info.push_grid;
  } else
  if (grid > tile_end - tile_begin) grid = tile_end - tile_begin;
  if (grid < 1) grid = 1;
  if (grid > kStatMaxCtas || plan->pair_push_grid > kStatMaxCtas) p.stats = 0;   // table has one row per CTA
  if (plan->pair_kernel && tile_begin == 0 && tile_end == total) {
    p.trace_tile_slots = 2 * ((p.m_tiles_local + 1) / 2) * p.n_tiles_local * p.owners;
    // (an all-gather-pushing launch has a fixed grid: the consumers count its CTAs)
    // A launch that pushes the A operand trades one operand stage for the bounce ring its
    // communication warps copy through.
    TCCL_CHECK_CUDA(launch_fused_gemm_pair(p, ag_push ? plan->pair_push_grid : plan->pair_grid,
                                           reinterpret_cast<cudaStream_t>(stream),
                                           ag_push && p.ag_mc_dst == 0));
    return kOk;
  }
  p.trace_tile_slots = total;
  TCCL_CHECK_CUDA(launch_fused_gemm(p, grid, reinterpret_cast<cudaStream_t>(stream)));
  return kOk;
}

extern "C" int tccl_gemm_plan_launch_streamed(void* plan_, uint32_t epoch, uint32_t a_gate_target,
                                              int32_t flags, const TcclStreamChunk* chunks,
                                              int32_t n_chunks, uint64_t copy_stream_,
                                              uint64_t copy_stream2_, uint64_t stream_) {
  TCCL_CHECK_ARG(plan_ != nullptr && chunks != nullptr && n_chunks >= 1, "bad argument");
  GemmPlan* plan = static_cast<GemmPlan*>(plan_);
  cudaStream_t copy_streams[2] = {reinterpret_cast<cudaStream_t>(copy_stream_),
                                  reinterpret_cast<cudaStream_t>(copy_stream2_)};
  const int n_copy_streams = copy_stream2_ != 0 && copy_stream2_ != copy_stream_ ? 2 : 1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  for (int c = 0; c < n_copy_streams; ++c)
    TCCL_CHECK_ARG(copy_streams[c] != stream, "a copy stream must differ from the launch stream");
  while (static_cast<int>(plan->events.size()) < n_chunks + 1) {
    cudaEvent_t e;
    TCCL_CHECK_CUDA(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
    plan->events.push_back(e);
  }
  if ((flags & 4) != 0 && plan->streamed_before) {
    // The caller promises that nothing else pending on `stream` touches A: the copies only
    // have to follow this plan's own previous streamed call (its last launch read A).
    for (int c = 0; c < n_copy_streams; ++c)
      TCCL_CHECK_CUDA(cudaStreamWaitEvent(copy_streams[c], plan->done_event, 0));
  } else {
    // Earlier work on `stream` may still read A: the copies wait for all of it.
    TCCL_CHECK_CUDA(cudaEventRecord(plan->events[n_chunks], stream));
    for (int c = 0; c < n_copy_streams; ++c)
      TCCL_CHECK_CUDA(cudaStreamWaitEvent(copy_streams[c], plan->events[n_chunks], 0));
  }
  for (int i = 0; i < n_chunks; ++i) {
    const TcclStreamChunk& c = chunks[i];
    cudaStream_t copy_stream = copy_streams[i % n_copy_streams];
    TCCL_CHECK_ARG(c.n_ranges >= 0 && c.n_ranges <= TCCL_STREAM_MAX_RANGES, "too many ranges");
    for (int r = 0; r < c.n_ranges; ++r)
      TCCL_CHECK_CUDA(cudaMemcpyAsync(reinterpret_cast<void*>(c.dst[r]),
                                      reinterpret_cast<const void*>(c.src[r]), c.bytes[r],
                                      cudaMemcpyHostToDevice, copy_stream));
    TCCL_CHECK_CUDA(cudaEventRecord(plan->events[i], copy_stream));
    TCCL_CHECK_CUDA(cudaStreamWaitEvent(stream, plan->events[i], 0));
    int f = 0;
    if (i == n_chunks - 1) f |= flags & 1;
    if (i == 0) f |= flags & (2 | 8);
    int rc = tccl_gemm_plan_launch(plan_, epoch, a_gate_target, c.tile_begin, c.tile_end, f,
                                   stream_);
    if (rc != kOk) return rc;
  }
  if (plan->done_event == nullptr)
    TCCL_CHECK_CUDA(cudaEventCreateWithFlags(&plan->done_event, cudaEventDisableTiming));
  TCCL_CHECK_CUDA(cudaEventRecord(plan->done_event, stream));
  plan->streamed_before = true;
  return kOk;
}

extern "C" int tccl_gemm_plan_destroy(void* plan) {
  delete static_cast<GemmPlan*>(plan);
  return kOk;
}

extern "C" int tccl_wait_groups(uint64_t sig, int32_t sig_stride, int32_t n_src, int32_t n_groups,
                                uint64_t per_epoch, uint32_t epoch, int32_t skip_src,
                                uint64_t status, uint64_t budget_ns, int32_t rank,
                                uint64_t stream) {
  TCCL_CHECK_ARG(sig != 0 && per_epoch != 0, "null argument");
  TCCL_CHECK_CUDA(launch_wait_groups(reinterpret_cast<const uint32_t*>(sig), sig_stride, n_src,
                                     n_groups, reinterpret_cast<const uint32_t*>(per_epoch), epoch,
                                     skip_src,
                                     reinterpret_cast<uint32_t*>(status),
                                     budget_ns ? budget_ns : 2000000000ull, rank,
                                     reinterpret_cast<cudaStream_t>(stream)));
  return kOk;
}

// Loads every kernel of the library onto the current device.  With CUDA's lazy module
// loading the first launch of a kernel may have to wait for kernels already running on
// the device; a kernel that spins on a peer whose launch sits behind such a first launch
// (several ranks driven by one host thread) would then run into its wait budget.  Called
// once per device when a context is created.
extern "C" int tccl_preload_kernels(void) {
  using namespace tileccl;
  TCCL_CHECK_CUDA(preload_gemm_kernels());
  TCCL_CHECK_CUDA(preload_collective_kernels());
  TCCL_CHECK_CUDA(preload_push_kernels());
  TCCL_CHECK_CUDA(preload_prim_kernels());
  return kOk;
}
