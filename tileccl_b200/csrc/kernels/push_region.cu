// Pushes a rectangular region of a row-major matrix (rows x row_bytes at a pitch
// of ld_bytes) from this rank's heap to the same place in every peer's heap,
// row band by row band.  It is the communication half of the two-kernel overlap
// patterns of GEMM + all-scatter:
//   bulk_sync          GEMM kernel, then this kernel (stream order)
//   producer_consumer  GEMM kernel on one stream signals a local counter per row
//                      band; this kernel, on a second stream, waits for a band's
//                      counter before it pushes the band
// (reference: tileccl/patterns/bulk_sync.py:240-299 and
// tileccl/patterns/producer_consumer.py:328-393).  The consumer only ever waits
// on the producer of the SAME GPU, which never waits on it, and it is launched
// after the producer.
//
// Completion follows the three-phase counter protocol of the tile collectives
// (announce / move + publish / wait), see collectives.cu.
#include <cuda_runtime.h>

#include "../api.h"
#include "../device/ptx.cuh"
#include "../device/tile_mem.cuh"
#include "../device/tile_sync.cuh"
#include "../runtime/errors.h"

namespace tileccl {

struct PushRegionParams {
  uint64_t region;        // local address of the region's first byte (on the heap)
  uint64_t mc_region;     // multicast alias of the same bytes (0 = per-peer stores)
  int64_t ld_bytes;
  int32_t rows, row_bytes;
  int32_t band_rows;      // rows per band (one producer TileGroup)
  int32_t rank, world_size;
  int64_t heap_stride;
  uint64_t band_ready;    // local uint32[bands] written by the producer, 0 = do not wait
  uint32_t band_target_per_epoch;
  uint64_t counters;      // collective counter block (ready[8], done[8], cta_done)
  uint32_t epoch;
  int32_t phase_mask;
  uint64_t status;
  uint64_t budget_ns;
};

__global__ void __launch_bounds__(256) push_region_kernel(const PushRegionParams p) {
  __shared__ uint32_t abort_word;
  __shared__ int is_last;
  __shared__ int band_ok;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  uint32_t* counters = reinterpret_cast<uint32_t*>(p.counters);
  uint32_t* status = reinterpret_cast<uint32_t*>(p.status);
  const int ws = p.world_size, rank = p.rank;

  auto peer_counter = [&](int r, int idx) {
    return reinterpret_cast<uint32_t*>(static_cast<int64_t>(p.counters) +
                                       static_cast<int64_t>(r - rank) * p.heap_stride) + idx;
  };

  if ((p.phase_mask & 1) && blockIdx.x == 0 && threadIdx.x < ws && threadIdx.x != rank)
    red_release_sys_add(peer_counter(threadIdx.x, rank), 1u);  // my region may be overwritten

  if (p.phase_mask & 2) {
    // every peer has entered the call (its copy of the region is ours to write)
    bool ok = true;
    if (threadIdx.x < ws && threadIdx.x != rank) {
      uint32_t seen = 0;
      if (!tile_wait_ge(counters + threadIdx.x, p.epoch, wb, &seen)) {
        report_status(status, kStatusTimeoutSignal, 70, p.epoch, seen, rank, threadIdx.x);
        abort_word = 1;
      }
    }
    __syncthreads();
    ok = abort_word == 0;
    const int bands = (p.rows + p.band_rows - 1) / p.band_rows;
    const int vec_per_row = p.row_bytes >> 4;
    for (int b = blockIdx.x; ok && b < bands; b += gridDim.x) {
      if (p.band_ready != 0) {
        if (threadIdx.x == 0) {
          uint32_t seen = 0;
          const uint32_t target = p.band_target_per_epoch * p.epoch;
          band_ok = tile_wait_ge(reinterpret_cast<const uint32_t*>(p.band_ready) + b, target, wb,
                                 &seen)
                        ? 1
                        : 0;
          if (!band_ok) report_status(status, kStatusTimeoutSignal, 71, target, seen, rank, b);
        }
        __syncthreads();
        if (!band_ok) break;
      }
      const int row0 = b * p.band_rows;
      const int nrows = p.rows - row0 < p.band_rows ? p.rows - row0 : p.band_rows;
      const int total = nrows * vec_per_row;
      for (int i = threadIdx.x; i < total; i += blockDim.x) {
        const int r = i / vec_per_row, c = i - r * vec_per_row;
        const int64_t off = static_cast<int64_t>(row0 + r) * p.ld_bytes + (c << 4);
        const uint4 v = ld_remote_v4(reinterpret_cast<const char*>(p.region) + off);
        if (p.mc_region != 0) {
          multimem_st_v4(reinterpret_cast<char*>(p.mc_region) + off, v);
        } else {
          for (int d = 1; d < ws; ++d) {
            const int pr = (rank + d) % ws;
            st_remote_v4(reinterpret_cast<char*>(static_cast<int64_t>(p.region) +
                                                 static_cast<int64_t>(pr - rank) * p.heap_stride) +
                             off, v);
          }
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(counters + 16, 1u);
      is_last = (old == gridDim.x - 1) ? 1 : 0;
      if (is_last) counters[16] = 0;
    }
    __syncthreads();
    if (is_last && threadIdx.x < ws && threadIdx.x != rank) {
      __threadfence_system();
      red_release_sys_add(peer_counter(threadIdx.x, 8 + rank), 1u);
    }
  }

  if ((p.phase_mask & 4) && blockIdx.x == 0 && threadIdx.x < ws && threadIdx.x != rank) {
    uint32_t seen = 0;
    if (!tile_wait_ge(counters + 8 + threadIdx.x, p.epoch, wb, &seen))
      report_status(status, kStatusTimeoutSignal, 72, p.epoch, seen, rank, threadIdx.x);
  }
}

}  // namespace tileccl

using namespace tileccl;

extern "C" int tccl_push_region(uint64_t region, uint64_t mc_region, int64_t ld_bytes, int32_t rows,
                                int32_t row_bytes, int32_t band_rows, int32_t rank,
                                int32_t world_size, int64_t heap_stride, uint64_t band_ready,
                                uint32_t band_target_per_epoch, uint64_t counters, uint32_t epoch,
                                int32_t phase_mask, int32_t grid, uint64_t status,
                                uint64_t budget_ns, uint64_t stream) {
  TCCL_CHECK_ARG(region != 0 && counters != 0, "null argument");
  TCCL_CHECK_ARG(rows > 0 && row_bytes > 0 && band_rows > 0 && grid > 0, "empty region");
  TCCL_CHECK_ARG(region % 16 == 0 && ld_bytes % 16 == 0 && row_bytes % 16 == 0,
                 "region must be 16-byte aligned in base, pitch and width");
  TCCL_CHECK_ARG(world_size >= 1 && world_size <= TCCL_MAX_RANKS && rank >= 0 && rank < world_size,
                 "bad rank / world_size");
  PushRegionParams p;
  p.region = region; p.mc_region = mc_region; p.ld_bytes = ld_bytes; p.rows = rows;
  p.row_bytes = row_bytes; p.band_rows = band_rows; p.rank = rank; p.world_size = world_size;
  p.heap_stride = heap_stride; p.band_ready = band_ready;
  p.band_target_per_epoch = band_target_per_epoch; p.counters = counters; p.epoch = epoch;
  p.phase_mask = phase_mask; p.status = status;
  p.budget_ns = budget_ns ? budget_ns : 2000000000ull;
  push_region_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(p);
  TCCL_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

namespace tileccl {
cudaError_t preload_push_kernels() {
  cudaFuncAttributes a;
  return cudaFuncGetAttributes(&a, push_region_kernel);
}
}  // namespace tileccl
