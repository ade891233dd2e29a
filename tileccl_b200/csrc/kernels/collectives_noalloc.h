// In-place sum all-reduce over buffers that live on ONE GPU, without a single
// memory allocation.  This entry point has no counterpart in the reference
// library; it exists for callers that are not allowed to allocate device memory.
//
// Who cannot allocate: code that runs inside a region where the CUDA allocator
// is off limits - a process whose device memory is handed out once by its own
// pool and then frozen, a latency-critical serving loop that forbids anything
// that may synchronise the device, a plug-in that is given buffers by its host
// application and nothing else.  cudaMalloc / cudaFree may block, synchronise
// the whole device or fail under memory pressure; the ordinary all-reduce of
// this library takes its staging area and counters from the symmetric heap,
// i.e. it needs an allocation the first time a message size is seen.
//
// Here the scratch memory (staging copies of the operands and the arrival
// counters of the one-shot all-reduce kernel) is a fixed array that is part of
// the library image itself.  Every GPU that loads the library holds that array
// (TCCL_NOALLOC_SCRATCH_BYTES, about 4 MiB) until the process exits.
//
// Semantics: buffers[0 .. n_ranks) are `count` elements each, on the current
// device, 16-byte aligned; on return (stream order) every buffer holds the
// element-wise sum of all of them, accumulated in fp32 in buffer order.  It is
// the same kernel (allreduce_oneshot_kernel) the heap-based all-reduce uses for
// small messages, run once per emulated rank and phase.
//
// Limits and rules:
//   * n_ranks <= TCCL_NOALLOC_MAX_RANKS, count * element size <= TCCL_NOALLOC_MAX_BYTES;
//     larger requests are rejected with an error, nothing is launched.
//   * The first call on a device looks up the device address of the scratch
//     array (cudaGetSymbolAddress) with that device current.  Make that first
//     call before any stream capture begins.
//   * All calls on a device share the one scratch array, and it keeps what the
//     previous call left in it.  The words that must start at zero are cleared
//     on the stream at the start of every call.  Two calls that overlap on the
//     GPU (different streams, no dependency between them) race on the scratch
//     and give wrong results: serialise them.
//   * No cudaMalloc, cudaFree or allocating library routine is called.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TCCL_NOALLOC_MAX_RANKS 8
#define TCCL_NOALLOC_MAX_BYTES (256 * 1024)
// per rank: two staging parities + one counter block
#define TCCL_NOALLOC_RANK_BYTES (2 * TCCL_NOALLOC_MAX_BYTES + 256)
#define TCCL_NOALLOC_SCRATCH_BYTES (TCCL_NOALLOC_MAX_RANKS * TCCL_NOALLOC_RANK_BYTES)

// dtype: 0 fp16, 1 bf16, 2 fp32.  Returns 0 on success; on failure a non-zero
// code, with the reason available from tccl_last_error().
int tccl_allreduce_sum_noalloc(const uint64_t* buffers, int32_t n_ranks, int32_t dtype,
                               uint64_t count, uint64_t stream);

#ifdef __cplusplus
}
#endif
