// Low-latency ("LL") transport for small messages: every 16-byte line that
// crosses NVLink carries 8 bytes of payload and two copies of a 32-bit flag
// {data0, flag, data1, flag}.  The receiver polls the line itself until both flags
// equal the value of the current call, so data and "data is here" arrive in the
// same store: no fence, no separate signal, no announcement round.  Half of the
// wire bytes are flags, which is the right trade below ~64 KiB where a call is
// latency-bound.  (A 16-byte store is performed as two 8-byte halves at worst,
// and each half carries its own flag.)
//
// Lines land in a library-owned staging area on the receiver, double-buffered by
// the parity of the call number; a receiver acknowledges each source once it has
// consumed its lines, and a sender does not reuse a parity before the matching
// acknowledgement of two calls ago has arrived (bounded wait).
#pragma once
#include "tile_sync.cuh"

namespace tileccl {

static constexpr uint32_t kLLMaxBytes = 1024 * 1024;        // payload per (source, destination)
static constexpr uint32_t kLLLineBytes = 16;                // 8 payload bytes per line
// A staging slot holds the lines of one (source, destination) message: 2 bytes of staging
// per payload byte.  The slot size is a launch parameter (the host sizes the staging for the
// message class in use), at least kLLMinSlotBytes.
static constexpr uint64_t kLLMinSlotBytes = 128 * 1024;

__device__ __forceinline__ void ll_store_line(void* line, uint32_t d0, uint32_t d1, uint32_t flag) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(line), "r"(d0), "r"(flag),
               "r"(d1), "r"(flag)
               : "memory");
}

// Polls `line` until both flags equal `flag`; false on time-out.
__device__ __forceinline__ bool ll_load_line(const void* line, uint32_t flag, uint32_t& d0,
                                             uint32_t& d1, const WaitBudget& wb) {
  for (uint32_t it = 0;; ++it) {
    uint32_t f0, f1;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(d0), "=r"(f0), "=r"(d1), "=r"(f1)
                 : "l"(line)
                 : "memory");
    if (f0 == flag && f1 == flag) return true;
    if (wb.expired(it)) return false;
  }
}

// Sends `bytes` (a multiple of 8, 8-byte aligned source) as LL lines to `dst_lines`.
__device__ __forceinline__ void ll_send(char* dst_lines, const char* src, uint32_t bytes,
                                        uint32_t flag, uint32_t tid, uint32_t nthreads) {
  const uint32_t lines = bytes >> 3;
  for (uint32_t i = tid; i < lines; i += nthreads) {
    const uint2 v = *reinterpret_cast<const uint2*>(src + (static_cast<uint64_t>(i) << 3));
    ll_store_line(dst_lines + static_cast<uint64_t>(i) * kLLLineBytes, v.x, v.y, flag);
  }
}

// Receives `bytes` from local LL lines into `dst` (8-byte aligned).  Returns false when a
// line never arrived within the budget.
__device__ __forceinline__ bool ll_recv(char* dst, const char* lines_local, uint32_t bytes,
                                        uint32_t flag, uint32_t tid, uint32_t nthreads,
                                        const WaitBudget& wb) {
  const uint32_t lines = bytes >> 3;
  bool ok = true;
  for (uint32_t i = tid; i < lines && ok; i += nthreads) {
    uint32_t d0, d1;
    ok = ll_load_line(lines_local + static_cast<uint64_t>(i) * kLLLineBytes, flag, d0, d1, wb);
    if (ok) *reinterpret_cast<uint2*>(dst + (static_cast<uint64_t>(i) << 3)) = make_uint2(d0, d1);
  }
  return ok;
}

}  // namespace tileccl
