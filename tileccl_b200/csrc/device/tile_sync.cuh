// Cross-GPU synchronisation primitives: release/acquire flags, counters,
// credits, remote atomics and a multi-rank barrier, all at system scope and all
// with bounded waits.  Names follow the reference's device API
// (tileccl/sync/primitives.py:62-568, tileccl_v2/ipc.py:136-254); the
// differences are deliberate:
//   * every wait takes a WaitBudget and returns false on time-out instead of
//     spinning for ever (the reference only bounds tile_try_wait);
//   * counters are monotonic ("epoch-valued"), so nothing is reset between calls.
#pragma once
#include "ptx.cuh"
#include "symm_ptr.cuh"

namespace tileccl {

// --- raw system-scope accessors -------------------------------------------
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void fence_acq_rel_sys() {
  asm volatile("fence.acq_rel.sys;" ::: "memory");
}

// --- remote atomics (acq_rel, system scope) -------------------------------
// `target` is a pointer into the *caller's* heap; the operation is applied to
// the same object in `to_rank`'s heap.
#define TILECCL_ATOMIC(NAME, PTXOP, TYPE, PTXT)                                             \
  __device__ __forceinline__ TYPE tile_atomic_##NAME(const SymmWindow& w, TYPE* target,     \
                                                     TYPE value, int to_rank) {             \
    TYPE* p = translate_ptr(w, target, w.rank, to_rank);                                    \
    TYPE old;                                                                               \
    asm volatile("atom.acq_rel.sys.global." PTXOP "." PTXT " %0, [%1], %2;"                 \
                 : "=r"(old)                                                                \
                 : "l"(p), "r"(value)                                                       \
                 : "memory");                                                               \
    return old;                                                                             \
  }
TILECCL_ATOMIC(add, "add", uint32_t, "u32")
TILECCL_ATOMIC(xchg, "exch", uint32_t, "b32")
TILECCL_ATOMIC(min, "min", uint32_t, "u32")
TILECCL_ATOMIC(max, "max", uint32_t, "u32")
TILECCL_ATOMIC(and, "and", uint32_t, "b32")
TILECCL_ATOMIC(or, "or", uint32_t, "b32")
TILECCL_ATOMIC(xor, "xor", uint32_t, "b32")
#undef TILECCL_ATOMIC

__device__ __forceinline__ uint32_t tile_atomic_cas(const SymmWindow& w, uint32_t* target,
                                                    uint32_t compare, uint32_t value,
                                                    int to_rank) {
  uint32_t* p = translate_ptr(w, target, w.rank, to_rank);
  uint32_t old;
  asm volatile("atom.acq_rel.sys.global.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old)
               : "l"(p), "r"(compare), "r"(value)
               : "memory");
  return old;
}

// --- binary flags ----------------------------------------------------------
// Producer: publish everything written before this call, then raise the flag
// in `to_rank`'s heap.
__device__ __forceinline__ void tile_signal(const SymmWindow& w, uint32_t* flag, int to_rank) {
  st_release_sys(translate_ptr(w, flag, w.rank, to_rank), 1u);
}

// Consumer: wait for a local flag and consume it (1 -> 0): one consumer per flag.
__device__ __forceinline__ bool tile_wait(uint32_t* flag, const WaitBudget& wb) {
  for (uint32_t it = 0;; ++it) {
    uint32_t old;
    asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], 1, 0;"
                 : "=r"(old)
                 : "l"(flag)
                 : "memory");
    if (old == 1u) return true;
    if (wb.expired(it)) return false;
  }
}

// Bounded by a poll count instead of time; consumes on success.
__device__ __forceinline__ bool tile_try_wait(uint32_t* flag, int max_spins) {
  for (int it = 0; it < max_spins; ++it) {
    uint32_t old;
    asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], 1, 0;"
                 : "=r"(old)
                 : "l"(flag)
                 : "memory");
    if (old == 1u) return true;
  }
  return false;
}

// Non-consuming wait: any number of consumers may poll the same flag.
__device__ __forceinline__ bool tile_poll(const uint32_t* flag, const WaitBudget& wb) {
  for (uint32_t it = 0;; ++it) {
    if (ld_acquire_sys(flag) != 0u) return true;
    if (wb.expired(it)) return false;
  }
}
__device__ __forceinline__ bool tile_try_poll(const uint32_t* flag, int max_spins) {
  for (int it = 0; it < max_spins; ++it)
    if (ld_acquire_sys(flag) != 0u) return true;
  return false;
}

// --- counters --------------------------------------------------------------
__device__ __forceinline__ void tile_signal_add(const SymmWindow& w, uint32_t* counter,
                                                uint32_t amount, int to_rank) {
  red_release_sys_add(translate_ptr(w, counter, w.rank, to_rank), amount);
}

// Wait until a local counter has reached `target` (wrap-safe signed compare).
// On time-out, `*observed` holds the last value seen.
__device__ __forceinline__ bool tile_wait_ge(const uint32_t* counter, uint32_t target,
                                             const WaitBudget& wb, uint32_t* observed = nullptr) {
  uint32_t v = 0;
  for (uint32_t it = 0;; ++it) {
    v = ld_acquire_sys(counter);
    if (static_cast<int32_t>(v - target) >= 0) return true;
    if (wb.expired(it)) {
      if (observed) *observed = v;
      return false;
    }
    if (it > 64) __nanosleep(64);
  }
}

// --- credits (flow control) -----------------------------------------------
// A producer takes one credit from a local pool before sending; the consumer
// gives it back remotely when the slot may be reused.
__device__ __forceinline__ bool tile_acquire_credit(uint32_t* credits, const WaitBudget& wb) {
  for (uint32_t it = 0;; ++it) {
    uint32_t cur = ld_acquire_sys(credits);
    if (cur > 0u) {
      uint32_t old;
      asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], %2, %3;"
                   : "=r"(old)
                   : "l"(credits), "r"(cur), "r"(cur - 1u)
                   : "memory");
      if (old == cur) return true;
    }
    if (wb.expired(it)) return false;
  }
}
__device__ __forceinline__ void tile_release_credit(const SymmWindow& w, uint32_t* credits,
                                                    int to_rank) {
  red_release_sys_add(translate_ptr(w, credits, w.rank, to_rank), 1u);
}

// --- multi-rank barrier ----------------------------------------------------
// One thread per rank calls this.  `counter` is a symmetric uint32 that only
// grows: each rank adds 1 to the counter of every rank and then waits until its
// own copy reaches `epoch * world_size` (epoch = 1, 2, 3 ... per use).
__device__ __forceinline__ bool tile_barrier(const SymmWindow& w, uint32_t* counter,
                                             uint32_t epoch, const WaitBudget& wb) {
  fence_acq_rel_sys();
  for (int r = 0; r < w.world_size; ++r)
    red_release_sys_add(translate_ptr(w, counter, w.rank, r), 1u);
  return tile_wait_ge(counter, epoch * static_cast<uint32_t>(w.world_size), wb);
}

}  // namespace tileccl
