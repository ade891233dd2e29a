// Symmetric-heap addressing on the device.
//
// Every rank's heap is mapped into one contiguous virtual window of
// `world_size * stride` bytes, rank r at `base + r * stride`, in every process.
// Translating a pointer from one rank's heap to another's is therefore pure
// arithmetic (the reference needs two table loads per translation,
// tileccl/memory/translation.py:73-92).  When an NVLS multicast object is bound,
// `mc_base` is the multicast alias of the heap: an address `mc_base + offset`
// names `offset` in every rank's heap at once (multimem.* instructions only).
#pragma once
#include <stdint.h>

namespace tileccl {

struct SymmWindow {
  uint64_t base;      // address of rank 0's heap in this process
  uint64_t stride;    // bytes between consecutive ranks' heaps (= heap size)
  uint64_t mc_base;   // multicast alias of the heap, 0 when NVLS is not bound
  int32_t rank;       // calling rank
  int32_t world_size;
};

__host__ __device__ __forceinline__ uint64_t symm_heap_base(const SymmWindow& w, int rank) {
  return w.base + static_cast<uint64_t>(rank) * w.stride;
}

// Offset of a local-heap pointer inside its heap.
template <typename T>
__host__ __device__ __forceinline__ uint64_t symm_offset(const SymmWindow& w, const T* p,
                                                         int owner_rank) {
  return reinterpret_cast<uint64_t>(p) - symm_heap_base(w, owner_rank);
}

// --- debug build: recorded bounds checks -----------------------------------
// Compiled with -DTILECCL_DEBUG_CHECKS every translation and every symmetric tile or
// span an accessor is about to touch is checked against the heap window.  A violation
// is RECORDED (the first one per translation unit wins, `count` keeps counting) and the
// access is redirected to the caller's own copy (translate_ptr) or skipped (the tile
// verbs and collectives), so the kernel runs to its end and the context stays usable:
// nothing traps.  The host reads the record with the reader a translation unit defines
// through TILECCL_DEFINE_DEBUG_READER.  The reference has no sanitizer of its own; its
// safety is by protocol design only.
struct DebugRecord {
  uint32_t count;      // violations seen since the last clear
  uint32_t code;       // DebugCode of the first one
  int32_t rank;        // calling rank
  int32_t from_rank;   // owner the address was claimed to belong to
  int32_t to_rank;     // target rank of the translation (-1 for a span check)
  uint32_t enabled;    // 1 in a debug build (filled by the reader)
  uint64_t addr;       // offending address
  uint64_t bytes;      // extent that was checked (0 for a bare translation)
};
enum DebugCode : uint32_t {
  kDebugBadRank = 1,        // from_rank / to_rank outside [0, world_size)
  kDebugOutsideHeap = 2,    // the address is not inside from_rank's heap
  kDebugSpanOutsideHeap = 3,// [addr, addr + bytes) leaves the owner's heap
  kDebugNoMulticast = 4,    // a multimem verb without a bound multicast mapping
};

#if defined(TILECCL_DEBUG_CHECKS) && defined(__CUDACC__)
static __device__ DebugRecord g_debug_record;   // one per translation unit

__device__ __forceinline__ void debug_report(uint32_t code, const SymmWindow& w, int from_rank,
                                             int to_rank, uint64_t addr, uint64_t bytes) {
  if (atomicAdd(&g_debug_record.count, 1u) == 0) {
    g_debug_record.code = code;
    g_debug_record.rank = w.rank;
    g_debug_record.from_rank = from_rank;
    g_debug_record.to_rank = to_rank;
    g_debug_record.addr = addr;
    g_debug_record.bytes = bytes;
  }
}
#define TILECCL_DEFINE_DEBUG_READER(fn)                                                        \
  extern "C" int fn(void* out, int clear) {                                                    \
    tileccl::DebugRecord r;                                                                    \
    cudaError_t e = cudaMemcpyFromSymbol(&r, tileccl::g_debug_record, sizeof(r));              \
    if (e != cudaSuccess) return static_cast<int>(e);                                          \
    r.enabled = 1;                                                                             \
    *static_cast<tileccl::DebugRecord*>(out) = r;                                              \
    if (clear && r.count != 0) {                                                               \
      tileccl::DebugRecord z = {};                                                             \
      e = cudaMemcpyToSymbol(tileccl::g_debug_record, &z, sizeof(z));                          \
    }                                                                                          \
    return static_cast<int>(e);                                                                \
  }
#else
#define TILECCL_DEFINE_DEBUG_READER(fn)                                                        \
  extern "C" int fn(void* out, int clear) {                                                    \
    (void)clear;                                                                               \
    tileccl::DebugRecord z = {};                                                               \
    *static_cast<tileccl::DebugRecord*>(out) = z;                                              \
    return 0;                                                                                  \
  }
#endif

// True when [p, p + bytes) lies inside `owner_rank`'s heap.  Always true in a release
// build (the check compiles away); in a debug build a violation is recorded.
template <typename T>
__host__ __device__ __forceinline__ bool symm_span_ok(const SymmWindow& w, const T* p,
                                                      uint64_t bytes, int owner_rank) {
#if defined(TILECCL_DEBUG_CHECKS) && defined(__CUDA_ARCH__)
  const uint64_t a = reinterpret_cast<uint64_t>(p);
  if (owner_rank < 0 || owner_rank >= w.world_size) {
    debug_report(kDebugBadRank, w, owner_rank, -1, a, bytes);
    return false;
  }
  const uint64_t off = a - symm_heap_base(w, owner_rank);
  if (off >= w.stride || bytes > w.stride - off) {
    debug_report(kDebugSpanOutsideHeap, w, owner_rank, -1, a, bytes);
    return false;
  }
#endif
  return true;
}

// Same object, in `to_rank`'s heap.  Only defined for pointers into the heap.
template <typename T>
__host__ __device__ __forceinline__ T* translate_ptr(const SymmWindow& w, T* p, int from_rank,
                                                     int to_rank) {
#if defined(TILECCL_DEBUG_CHECKS) && defined(__CUDA_ARCH__)
  const uint64_t a = reinterpret_cast<uint64_t>(p);
  if (from_rank < 0 || from_rank >= w.world_size || to_rank < 0 || to_rank >= w.world_size) {
    debug_report(kDebugBadRank, w, from_rank, to_rank, a, 0);
    return p;
  }
  if (a - symm_heap_base(w, from_rank) >= w.stride) {
    debug_report(kDebugOutsideHeap, w, from_rank, to_rank, a, 0);
    return p;
  }
#endif
  int64_t delta = (static_cast<int64_t>(to_rank) - static_cast<int64_t>(from_rank)) *
                  static_cast<int64_t>(w.stride);
  return reinterpret_cast<T*>(reinterpret_cast<uint64_t>(p) + static_cast<uint64_t>(delta));
}

// Multicast alias of a pointer into the calling rank's heap (nullptr if NVLS is off).
template <typename T>
__host__ __device__ __forceinline__ T* mc_ptr(const SymmWindow& w, T* p) {
  if (w.mc_base == 0) return nullptr;
  return reinterpret_cast<T*>(w.mc_base + symm_offset(w, p, w.rank));
}

// Debug-build guard of the multimem verbs: a mapping is bound and the span is inside the
// caller's heap.  Always true in a release build.
template <typename T>
__host__ __device__ __forceinline__ bool mc_span_ok(const SymmWindow& w, const T* p,
                                                    uint64_t bytes) {
#if defined(TILECCL_DEBUG_CHECKS) && defined(__CUDA_ARCH__)
  if (w.mc_base == 0) {
    debug_report(kDebugNoMulticast, w, w.rank, -1, reinterpret_cast<uint64_t>(p), bytes);
    return false;
  }
#endif
  return symm_span_ok(w, p, bytes, w.rank);
}

// --- 16-byte remote accessors ---------------------------------------------
// Loads bypass L1 (.cg) so data written by a peer over NVLink is never served
// from a stale L1 line; stores are plain global stores (write-through to L2 /
// the link).
__device__ __forceinline__ uint4 ld_remote_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.cg.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_remote_v4(void* p, const uint4& v) {
  asm volatile("st.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_stream_v4(const void* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

// --- NVLS (multimem) accessors: address must be a multicast alias ---------
__device__ __forceinline__ void multimem_st_v4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(mc),
               "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
// Sum over all ranks of 8 fp16 / 8 bf16 / 4 fp32 values, accumulated in fp32 in the switch.
__device__ __forceinline__ uint4 multimem_ld_reduce_f16x8(const void* mc) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_ld_reduce_f32x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ void multimem_red_add_u32(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}

}  // namespace tileccl
