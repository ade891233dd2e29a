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
#include "../device/tile_comm.cuh"
#include "../device/tile_compute.cuh"
#include "../device/tile_sync.cuh"
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
enum CollDtype : int { kF16 = 0, kBF16 = 1, kF32 = 2, kBytes = 3 };

// Counter block layout (uint32, on the symmetric heap):
//   [0, 8)   ready[src]    phase-1 announcements received from rank src
//   [8, 16)  done[src]     phase-2 completions received from rank src
//   [16]     cta_done      local: CTAs of the current launch that finished phase 2
static constexpr int kCollCounters = 32;
static constexpr int kMaxRanks = TCCL_MAX_RANKS;

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

template <typename T>
__device__ __forceinline__ T* peer(const CollParams& p, uint64_t local, int r) {
  return reinterpret_cast<T*>(local + static_cast<int64_t>(r - p.rank) * p.heap_stride);
}
template <typename T>
__device__ __forceinline__ T* mcast(const CollParams& p, uint64_t local) {
  return reinterpret_cast<T*>(p.mc_base + (local - p.heap_base));
}

__device__ __forceinline__ float4 as_f4(const uint4& v) {
  return make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z),
                     __uint_as_float(v.w));
}

// acc (8 floats for 16-bit types, 4 for fp32) += v
__device__ __forceinline__ void accumulate(int dtype, float* acc, const uint4& v) {
  if (dtype == kF32) {
    float4 f = as_f4(v);
    acc[0] += f.x; acc[1] += f.y; acc[2] += f.z; acc[3] += f.w;
  } else {
    tile_accumulate_16x8(dtype == kBF16, acc, v);
  }
}
__device__ __forceinline__ uint4 finish(int dtype, const float* acc) {
  if (dtype == kF32)
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]),
                      __float_as_uint(acc[3]));
  return tile_cast_f32x8(dtype == kBF16, acc);
}
__device__ __forceinline__ uint4 mc_reduce(int dtype, const void* mc) {
  return dtype == kF32 ? multimem_ld_reduce_f32x4(mc)
                       : dtype == kBF16 ? multimem_ld_reduce_bf16x8(mc)
                                        : multimem_ld_reduce_f16x8(mc);
}

// Grid-stride copy from local memory to one (possibly remote) destination.  Moves
// 16 bytes per access when both addresses and the length allow it; otherwise one
// element per access (chunk offsets of odd-sized messages are only element-aligned).
template <typename T>
__device__ __forceinline__ void copy_elems(char* dst, const char* src, uint64_t bytes) {
  const uint64_t n = bytes / sizeof(T);
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    reinterpret_cast<T*>(dst)[i] = reinterpret_cast<const T*>(src)[i];
}
__device__ __forceinline__ bool vec_ok(const void* a, const void* b, uint64_t bytes) {
  return ((reinterpret_cast<uint64_t>(a) | reinterpret_cast<uint64_t>(b) | bytes) & 15u) == 0;
}
__device__ __forceinline__ void copy_vec(char* dst, const char* src, uint64_t bytes, int es) {
  if (vec_ok(dst, src, bytes)) {
    // Eight 16-byte loads in flight per thread before the first store: the copy is bound by
    // the link, not by one load latency per store.
    constexpr int U = 8;
    const uint64_t n = bytes >> 4;
    const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
    uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    for (; i + (U - 1) * stride < n; i += U * stride) {
      uint4 v[U];
#pragma unroll
      for (int j = 0; j < U; ++j) v[j] = *reinterpret_cast<const uint4*>(src + ((i + j * stride) << 4));
#pragma unroll
      for (int j = 0; j < U; ++j) st_remote_v4(dst + ((i + j * stride) << 4), v[j]);
    }
    for (; i < n; i += stride)
      st_remote_v4(dst + (i << 4), *reinterpret_cast<const uint4*>(src + (i << 4)));
  } else if (es == 8) {
    copy_elems<uint64_t>(dst, src, bytes);
  } else if (es == 4) {
    copy_elems<uint32_t>(dst, src, bytes);
  } else if (es == 2) {
    copy_elems<uint16_t>(dst, src, bytes);
  } else {
    copy_elems<uint8_t>(dst, src, bytes);
  }
}
__device__ __forceinline__ void copy_vec_mc(char* mc_dst, const char* src, uint64_t bytes) {
  constexpr int U = 8;
  const uint64_t n = bytes >> 4;
  const uint64_t stride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  uint64_t i = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < n; i += U * stride) {
    uint4 v[U];
#pragma unroll
    for (int j = 0; j < U; ++j) v[j] = *reinterpret_cast<const uint4*>(src + ((i + j * stride) << 4));
#pragma unroll
    for (int j = 0; j < U; ++j) multimem_st_v4(mc_dst + ((i + j * stride) << 4), v[j]);
  }
  for (; i < n; i += stride)
    multimem_st_v4(mc_dst + (i << 4), *reinterpret_cast<const uint4*>(src + (i << 4)));
}

// Wait until counter[r] >= epoch for every r in the dependency set (thread r polls).
__device__ __forceinline__ bool wait_all(const CollParams& p, const uint32_t* counters,
                                         int only_rank, const WaitBudget& wb, uint32_t where) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  const int r = threadIdx.x;
  if (r < p.world_size && r != p.rank && (only_rank < 0 || r == only_rank)) {
    uint32_t seen = 0;
    if (!tile_wait_ge(counters + r, p.epoch, wb, &seen)) {
      report_status(reinterpret_cast<uint32_t*>(p.status), kStatusTimeoutSignal, where, p.epoch,
                    seen, p.rank, r);
      failed = 1;
    }
  }
  __syncthreads();
  return failed == 0;
}

// counter[rank] += 1 in the heap of every rank of the dependency set.
__device__ __forceinline__ void signal_all(const CollParams& p, int offset, int only_rank) {
  uint32_t* c = reinterpret_cast<uint32_t*>(p.counters) + offset + p.rank;
  const int r = threadIdx.x;
  if (r < p.world_size && r != p.rank && (only_rank < 0 || r == only_rank))
    red_release_sys_add(peer<uint32_t>(p, reinterpret_cast<uint64_t>(c), r), 1u);
}

}  // namespace

__global__ void __launch_bounds__(512) collective_kernel(const CollParams p) {
  __shared__ uint32_t abort_word;
  __shared__ int is_last;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  uint32_t* counters = reinterpret_cast<uint32_t*>(p.counters);
  const uint32_t* ready = counters;
  const uint32_t* done = counters + 8;
  uint32_t* cta_done = counters + 16;
  const int ws = p.world_size, rank = p.rank;
  const bool rooted = p.op == kBroadcast || p.op == kScatter;
  const bool is_root = rank == p.root;

  // ---- phase 1: announce ---------------------------------------------------
  if ((p.phase_mask & 1) && blockIdx.x == 0) {
    // Everything this rank's stream did before the call is visible (kernel boundary);
    // a rooted op only needs receivers -> root, the others need all -> all.
    if (!rooted) signal_all(p, 0, -1);
    else if (!is_root) signal_all(p, 0, p.root);
  }

  // ---- phase 2: wait for dependencies, move data, publish ------------------
  if (p.phase_mask & 2) {
    bool ok = true;
    if (!rooted) ok = wait_all(p, ready, -1, wb, 60);
    else if (is_root) ok = wait_all(p, ready, -1, wb, 61);
    if (ok) {
      const char* src = reinterpret_cast<const char*>(p.src);
      char* dst = reinterpret_cast<char*>(p.dst);
      const uint64_t bytes = p.bytes;
      const uint64_t nvec = bytes >> 4;
      const uint64_t gstride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
      const uint64_t gtid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;

      if (p.op == kAllGather) {
        // own chunk -> slot `rank` of every rank's output
        if (p.use_multimem && (bytes & 15) == 0) {
          copy_vec_mc(mcast<char>(p, p.dst) + rank * bytes, src, bytes);
        } else {
          for (int d = 0; d < ws; ++d) {
            const int r = (rank + d) % ws;
            copy_vec(peer<char>(p, p.dst, r) + rank * bytes, src, bytes, p.elem_size);
          }
        }
      } else if (p.op == kBroadcast) {
        if (is_root) {
          if (p.use_multimem && (bytes & 15) == 0) {
            copy_vec_mc(mcast<char>(p, p.dst), src, bytes);
          } else {
            for (int d = 1; d < ws; ++d)
              copy_vec(peer<char>(p, p.dst, (rank + d) % ws), src, bytes, p.elem_size);
          }
        }
      } else if (p.op == kScatter) {
        if (is_root) {
          for (int d = 0; d < ws; ++d) {
            const int r = (rank + d) % ws;
            copy_vec(peer<char>(p, p.dst, r), src + r * bytes, bytes, p.elem_size);
          }
        }
      } else if (p.op == kReduceScatter || p.op == kAllReduceTwoShot) {
        // Reduce chunk `rank` over all ranks.  reduce-scatter: chunk = bytes, output to dst.
        // all-reduce: buffer split into ws chunks of `chunk` bytes (16-byte multiple); the
        // reduced chunk is pushed back into every rank's buffer.
        uint64_t chunk = bytes, chunk_off = rank * bytes, my_bytes = bytes;
        if (p.op == kAllReduceTwoShot) {
          chunk = ((bytes + ws - 1) / ws + 15) & ~static_cast<uint64_t>(15);
          chunk_off = rank * chunk;
          my_bytes = chunk_off >= bytes ? 0 : (bytes - chunk_off < chunk ? bytes - chunk_off : chunk);
        }
        // Chunk offsets of a reduce-scatter are only element-aligned when the chunk is not a
        // multiple of 16 bytes: then everything goes through the scalar loop below.
        const bool aligned = ((chunk_off | reinterpret_cast<uint64_t>(dst)) & 15u) == 0;
        const uint64_t n = aligned ? (my_bytes >> 4) : 0;
        uint64_t i = gtid;
        if (p.use_multimem) {
          // In-switch reduction: several multimem.ld_reduce in flight per thread, then the
          // stores (one multimem.st reaches every rank).
          constexpr int U = 4;
          for (; i + (U - 1) * gstride < n; i += U * gstride) {
            uint4 o[U];
#pragma unroll
            for (int j = 0; j < U; ++j)
              o[j] = mc_reduce(p.dtype, mcast<char>(p, p.src) + chunk_off + ((i + j * gstride) << 4));
#pragma unroll
            for (int j = 0; j < U; ++j) {
              const uint64_t ii = i + j * gstride;
              if (p.op == kReduceScatter) *reinterpret_cast<uint4*>(dst + (ii << 4)) = o[j];
              else multimem_st_v4(mcast<char>(p, p.dst) + chunk_off + (ii << 4), o[j]);
            }
          }
        }
        if (!p.use_multimem) {
          // Peer loads of two items in flight per thread before the first accumulate.
          for (; i + gstride < n; i += 2 * gstride) {
            uint4 v0[kMaxRanks], v1[kMaxRanks];
            const uint64_t off0 = chunk_off + (i << 4), off1 = chunk_off + ((i + gstride) << 4);
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < ws) {
                v0[r] = ld_remote_v4(peer<char>(p, p.src, r) + off0);
                v1[r] = ld_remote_v4(peer<char>(p, p.src, r) + off1);
              }
            float a0[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float a1[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < ws) {
                accumulate(p.dtype, a0, v0[r]);
                accumulate(p.dtype, a1, v1[r]);
              }
            const uint4 o0 = finish(p.dtype, a0), o1 = finish(p.dtype, a1);
            if (p.op == kReduceScatter) {
              *reinterpret_cast<uint4*>(dst + (i << 4)) = o0;
              *reinterpret_cast<uint4*>(dst + ((i + gstride) << 4)) = o1;
            } else {
#pragma unroll
              for (int r = 0; r < kMaxRanks; ++r)
                if (r < ws) {
                  st_remote_v4(peer<char>(p, p.dst, r) + off0, o0);
                  st_remote_v4(peer<char>(p, p.dst, r) + off1, o1);
                }
            }
          }
        }
        for (; i < n; i += gstride) {
          uint4 out;
          const uint64_t off = chunk_off + (i << 4);
          if (p.use_multimem) {
            out = mc_reduce(p.dtype, mcast<char>(p, p.src) + off);
          } else {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            uint4 v[kMaxRanks];
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < ws) v[r] = ld_remote_v4(peer<char>(p, p.src, r) + off);
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < ws) accumulate(p.dtype, acc, v[r]);
            out = finish(p.dtype, acc);
          }
          if (p.op == kReduceScatter) {
            *reinterpret_cast<uint4*>(dst + (i << 4)) = out;
          } else if (p.use_multimem) {
            multimem_st_v4(mcast<char>(p, p.dst) + off, out);
          } else {
#pragma unroll
            for (int r = 0; r < kMaxRanks; ++r)
              if (r < ws) st_remote_v4(peer<char>(p, p.dst, r) + off, out);
          }
        }
        // scalar remainder: the < 16-byte tail, or the whole chunk when it is unaligned
        if ((n << 4) < my_bytes) {
          const int es = p.dtype == kF32 ? 4 : 2;
          for (uint64_t b = (n << 4) + gtid * es; b < my_bytes; b += gstride * es) {
            float a = 0.f;
            for (int r = 0; r < ws; ++r) {
              const char* q = peer<char>(p, p.src, r) + chunk_off + b;
              a += p.dtype == kF32 ? *reinterpret_cast<const volatile float*>(q)
                   : p.dtype == kBF16
                       ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(q))
                       : __half2float(*reinterpret_cast<const __half*>(q));
            }
            for (int r = 0; r < ws; ++r) {
              char* q = p.op == kReduceScatter ? dst + b : peer<char>(p, p.dst, r) + chunk_off + b;
              if (p.dtype == kF32) *reinterpret_cast<float*>(q) = a;
              else if (p.dtype == kBF16) *reinterpret_cast<__nv_bfloat16*>(q) = __float2bfloat16(a);
              else *reinterpret_cast<__half*>(q) = __float2half(a);
              if (p.op == kReduceScatter) break;
            }
          }
        }
      }
      // (kAllReduceOneShot moves its data in the dedicated kernel below.)
    }

    // publish: the last CTA to get here tells the peers that depend on this rank
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(cta_done, 1u);
      is_last = (old == gridDim.x - 1) ? 1 : 0;
      if (is_last) *cta_done = 0;
    }
    __syncthreads();
    if (is_last) {
      __threadfence_system();
      if (!rooted) signal_all(p, 8, -1);
      else if (is_root) signal_all(p, 8, -1);
    }
  }

  // ---- phase 3: wait for the completions this rank depends on --------------
  if ((p.phase_mask & 4) && blockIdx.x == 0) {
    if (!rooted) wait_all(p, done, -1, wb, 62);
    else if (!is_root) wait_all(p, done, p.root, wb, 63);
  }
}

// One-shot all-reduce for small messages: every rank publishes a copy of its
// buffer in a staging slot (double-buffered by epoch parity, so no exit barrier
// is needed), then sums all ranks' copies straight into its own buffer.
__global__ void __launch_bounds__(512) allreduce_oneshot_kernel(const CollParams p) {
  __shared__ uint32_t abort_word;
  __shared__ int is_last;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(p.budget_ns, &abort_word);
  uint32_t* counters = reinterpret_cast<uint32_t*>(p.counters);
  uint32_t* cta_done = counters + 16;
  const int ws = p.world_size;
  const uint64_t bytes = p.bytes;
  const uint64_t slot =
      p.stage_slot != 0 ? p.stage_slot : (bytes + 15) & ~static_cast<uint64_t>(15);
  const uint64_t stage = p.staging + (p.epoch & 1u) * slot;
  const uint64_t n = bytes >> 4;
  const uint64_t gstride = static_cast<uint64_t>(gridDim.x) * blockDim.x;
  const uint64_t gtid = static_cast<uint64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  char* buf = reinterpret_cast<char*>(p.dst);

  if (p.phase_mask & 1) {
    // publish a snapshot of the local buffer, then announce it
    copy_vec(reinterpret_cast<char*>(stage), buf, bytes & ~static_cast<uint64_t>(15), 16);
    if ((bytes & 15) && gtid == 0)
      for (uint64_t b = bytes & ~static_cast<uint64_t>(15); b < bytes; ++b)
        reinterpret_cast<char*>(stage)[b] = buf[b];
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
      const uint32_t old = atomicAdd(cta_done, 1u);
      is_last = (old == gridDim.x - 1) ? 1 : 0;
      if (is_last) *cta_done = 0;
    }
    __syncthreads();
    if (is_last) {
      __threadfence_system();
      signal_all(p, 0, -1);
    }
  }
  if (p.phase_mask & 2) {
    if (!wait_all(p, counters, -1, wb, 64)) return;
    for (uint64_t i = gtid; i < n; i += gstride) {
      float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      uint4 v[kMaxRanks];
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < ws) v[r] = ld_remote_v4(peer<char>(p, stage, r) + (i << 4));
#pragma unroll
      for (int r = 0; r < kMaxRanks; ++r)
        if (r < ws) accumulate(p.dtype, acc, v[r]);
      *reinterpret_cast<uint4*>(buf + (i << 4)) = finish(p.dtype, acc);
    }
    if ((bytes & 15) && gtid == 0) {
      const int es = p.dtype == kF32 ? 4 : 2;
      for (uint64_t b = n << 4; b < bytes; b += es) {
        float a = 0.f;
        for (int r = 0; r < ws; ++r) {
          const char* q = peer<char>(p, stage, r) + b;
          a += p.dtype == kF32 ? *reinterpret_cast<const volatile float*>(q)
               : p.dtype == kBF16 ? __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(q))
                                  : __half2float(*reinterpret_cast<const __half*>(q));
        }
        if (p.dtype == kF32) *reinterpret_cast<float*>(buf + b) = a;
        else if (p.dtype == kBF16) *reinterpret_cast<__nv_bfloat16*>(buf + b) = __float2bfloat16(a);
        else *reinterpret_cast<__half*>(buf + b) = __float2half(a);
      }
    }
  }
}

}  // namespace tileccl

using namespace tileccl;

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

namespace tileccl {
cudaError_t preload_collective_kernels() {
  cudaFuncAttributes a;
  cudaError_t e = cudaFuncGetAttributes(&a, collective_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, allreduce_oneshot_kernel);
  return e;
}
}  // namespace tileccl
