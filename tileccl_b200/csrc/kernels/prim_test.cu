// Small kernels that exercise the device primitives one at a time, so that the
// Python test-suite can check pointer translation, remote load/store, put/get,
// the signal/wait family, remote atomics and the bounded-wait time-out path
// against host expectations.  Each launch acts as ONE rank (`window.rank`).
#include <cuda_runtime.h>

#include "../api.h"
#include "../device/tile_collectives.cuh"
#include "../runtime/errors.h"

namespace tileccl {

enum PrimOp : int {
  kPrimPut = 0,          // a: local src, b: symmetric dst, n bytes -> peer
  kPrimGet = 1,          // a: symmetric src (read from peer), b: local dst
  kPrimRemoteStore = 2,  // a: local src -> registers -> peer's b
  kPrimRemoteLoad = 3,   // peer's a -> registers -> local b
  kPrimSignal = 4,       // raise flag a on peer
  kPrimWait = 5,         // wait + consume local flag a        (result[0] = 1 ok / 0 timeout)
  kPrimPoll = 6,         // non-consuming wait on local flag a
  kPrimSignalAdd = 7,    // counter a on peer += value
  kPrimWaitGe = 8,       // wait local counter a >= value
  kPrimAtomic = 9,       // remote atomic `sub_op` on a with value; result[0] = old
  kPrimBarrier = 10,     // tile_barrier on counter a with epoch = value
  kPrimCredit = 11,      // sub_op 0: acquire from local pool a; 1: release to peer's pool a
  kPrimTryWait = 12,     // bounded by `value` polls
  kPrimTranslate = 13,   // result64[0] = translate_ptr(a, rank, peer)
  kPrimPutMc = 14,       // a: local src -> multicast alias of b
  kPrimGetReduce = 15,   // multimem.ld_reduce over a -> local b (sub_op = dtype kind)
};

struct PrimArgs {
  SymmWindow w;
  int32_t op, sub_op, peer;
  uint32_t value, value2;
  uint64_t a, b, n;
  uint64_t result;  // uint32[4] / uint64[2] in device memory
  uint64_t budget_ns;
};

__global__ void prim_test_kernel(const PrimArgs x) {
  __shared__ uint32_t abort_word;
  if (threadIdx.x == 0) abort_word = 0;
  __syncthreads();
  WaitBudget wb;
  wb.start(x.budget_ns, &abort_word);
  uint32_t* res = reinterpret_cast<uint32_t*>(x.result);
  const int tid = threadIdx.x, nt = blockDim.x;
  const int rows = 1;
  TileView va{reinterpret_cast<char*>(x.a), static_cast<int64_t>(x.n), rows, static_cast<int>(x.n)};
  TileView vb{reinterpret_cast<char*>(x.b), static_cast<int64_t>(x.n), rows, static_cast<int>(x.n)};
  switch (x.op) {
    case kPrimPut: tile_put(x.w, va, vb, x.peer, tid, nt); break;
    case kPrimGet: tile_get(x.w, va, vb, x.peer, tid, nt); break;
    case kPrimRemoteStore: {
      uint4 frag[4];
      tile_load(va, frag, tid, nt);
      tile_remote_store(x.w, vb, x.peer, frag, tid, nt);
      break;
    }
    case kPrimRemoteLoad: {
      uint4 frag[4];
      tile_remote_load(x.w, va, x.peer, frag, tid, nt);
      tile_store(vb, frag, tid, nt);
      break;
    }
    case kPrimPutMc: tile_put_mc(x.w, va, vb, tid, nt); break;
    case kPrimGetReduce: tile_get_reduce(x.w, va, vb, x.sub_op, tid, nt); break;
    default: break;
  }
  if (tid != 0) return;
  uint32_t* fa = reinterpret_cast<uint32_t*>(x.a);
  switch (x.op) {
    case kPrimSignal: tile_signal(x.w, fa, x.peer); break;
    case kPrimWait: res[0] = tile_wait(fa, wb) ? 1u : 0u; break;
    case kPrimPoll: res[0] = tile_poll(fa, wb) ? 1u : 0u; break;
    case kPrimTryWait: res[0] = tile_try_wait(fa, static_cast<int>(x.value)) ? 1u : 0u; break;
    case kPrimSignalAdd: tile_signal_add(x.w, fa, x.value, x.peer); break;
    case kPrimWaitGe: {
      uint32_t seen = 0;
      res[0] = tile_wait_ge(fa, x.value, wb, &seen) ? 1u : 0u;
      res[1] = seen;
      break;
    }
    case kPrimAtomic: {
      uint32_t old = 0;
      switch (x.sub_op) {
        case 0: old = tile_atomic_add(x.w, fa, x.value, x.peer); break;
        case 1: old = tile_atomic_cas(x.w, fa, x.value, x.value2, x.peer); break;
        case 2: old = tile_atomic_xchg(x.w, fa, x.value, x.peer); break;
        case 3: old = tile_atomic_min(x.w, fa, x.value, x.peer); break;
        case 4: old = tile_atomic_max(x.w, fa, x.value, x.peer); break;
        case 5: old = tile_atomic_and(x.w, fa, x.value, x.peer); break;
        case 6: old = tile_atomic_or(x.w, fa, x.value, x.peer); break;
        case 7: old = tile_atomic_xor(x.w, fa, x.value, x.peer); break;
        default: break;
      }
      res[0] = old;
      break;
    }
    case kPrimBarrier: res[0] = tile_barrier(x.w, fa, x.value, wb) ? 1u : 0u; break;
    case kPrimCredit:
      if (x.sub_op == 0) res[0] = tile_acquire_credit(fa, wb) ? 1u : 0u;
      else tile_release_credit(x.w, fa, x.peer);
      break;
    case kPrimTranslate:
      reinterpret_cast<uint64_t*>(x.result)[0] =
          reinterpret_cast<uint64_t>(translate_ptr(x.w, fa, x.w.rank, x.peer));
      break;
    default: break;
  }
}

// Grid-wide put (local a -> peer's b) or get (peer's a -> local b) of a large buffer with
// the same 16-byte accessors as tile_put / tile_get: the bandwidth side of the
// point-to-point benchmark.
__global__ void __launch_bounds__(512) p2p_copy_kernel(SymmWindow w, int direction, int peer,
                                                       uint64_t a, uint64_t b, uint64_t bytes) {
  const TileCoop grid = tile_coop_grid();
  if (direction == 0) {
    char* dst = translate_ptr(w, reinterpret_cast<char*>(b), w.rank, peer);
    coll_detail::copy_vec(dst, reinterpret_cast<const char*>(a), bytes, 16, grid);
  } else {
    const char* src = translate_ptr(w, reinterpret_cast<char*>(a), w.rank, peer);
    char* dst = reinterpret_cast<char*>(b);
    const uint64_t n = bytes >> 4;
    constexpr int kU = 8;
    uint64_t i = grid.tid;
    for (; i + (kU - 1) * grid.nthreads < n; i += kU * grid.nthreads) {
      uint4 v[kU];
#pragma unroll
      for (int j = 0; j < kU; ++j) v[j] = ld_remote_v4(src + ((i + j * grid.nthreads) << 4));
#pragma unroll
      for (int j = 0; j < kU; ++j)
        *reinterpret_cast<uint4*>(dst + ((i + j * grid.nthreads) << 4)) = v[j];
    }
    for (; i < n; i += grid.nthreads)
      *reinterpret_cast<uint4*>(dst + (i << 4)) = ld_remote_v4(src + (i << 4));
  }
}

}  // namespace tileccl

using namespace tileccl;

extern "C" int tccl_p2p_copy(int32_t direction, int32_t rank, int32_t world_size, int32_t peer,
                             uint64_t window_base, uint64_t stride, uint64_t a, uint64_t b,
                             uint64_t bytes, int32_t grid, uint64_t stream) {
  TCCL_CHECK_ARG(direction == 0 || direction == 1, "direction must be 0 (put) or 1 (get)");
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size && peer >= 0 && peer < world_size, "bad rank/peer");
  TCCL_CHECK_ARG(a % 16 == 0 && b % 16 == 0 && bytes % 16 == 0,
                 "buffers and size must be multiples of 16 bytes");
  TCCL_CHECK_ARG(grid >= 1, "grid must be >= 1");
  SymmWindow w;
  w.base = window_base; w.stride = stride; w.mc_base = 0; w.rank = rank; w.world_size = world_size;
  p2p_copy_kernel<<<grid, 512, 0, reinterpret_cast<cudaStream_t>(stream)>>>(w, direction, peer, a, b,
                                                                             bytes);
  TCCL_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

extern "C" int tccl_prim_test(int32_t op, int32_t sub_op, int32_t rank, int32_t world_size,
                              int32_t peer, uint64_t window_base, uint64_t stride, uint64_t mc_base,
                              uint64_t a, uint64_t b, uint64_t n, uint32_t value, uint32_t value2,
                              uint64_t result, uint64_t budget_ns, uint64_t stream) {
  TCCL_CHECK_ARG(rank >= 0 && rank < world_size && peer >= 0 && peer < world_size, "bad rank/peer");
  TCCL_CHECK_ARG(result != 0, "result buffer required");
  TCCL_CHECK_ARG(n <= 128 * 4 * 16, "at most 8 KiB per call");
  if (op == kPrimPutMc || op == kPrimGetReduce)
    TCCL_CHECK_ARG(mc_base != 0, "multimem primitives need a multicast mapping");
  PrimArgs x;
  x.w.base = window_base;
  x.w.stride = stride;
  x.w.mc_base = mc_base;
  x.w.rank = rank;
  x.w.world_size = world_size;
  x.op = op; x.sub_op = sub_op; x.peer = peer; x.value = value; x.value2 = value2;
  x.a = a; x.b = b; x.n = n; x.result = result;
  x.budget_ns = budget_ns ? budget_ns : 1000000000ull;
  prim_test_kernel<<<1, 128, 0, reinterpret_cast<cudaStream_t>(stream)>>>(x);
  TCCL_CHECK_CUDA(cudaGetLastError());
  return kOk;
}

TILECCL_DEFINE_DEBUG_READER(tccl_debug_read_primitives)

namespace tileccl {
cudaError_t preload_prim_kernels() {
  cudaFuncAttributes a;
  cudaError_t e = cudaFuncGetAttributes(&a, prim_test_kernel);
  if (e == cudaSuccess) e = cudaFuncGetAttributes(&a, p2p_copy_kernel);
  return e;
}
}  // namespace tileccl
