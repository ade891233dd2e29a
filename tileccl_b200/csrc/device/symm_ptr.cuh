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

// Same object, in `to_rank`'s heap.  Only defined for pointers into the heap.
template <typename T>
__host__ __device__ __forceinline__ T* translate_ptr(const SymmWindow& w, T* p, int from_rank,
                                                     int to_rank) {
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
