// Glue for kernels written outside the library (see tileccl_b200/userkernel.py):
// the argument block such a kernel receives and a macro that writes the
// `extern "C"` entry point the Python loader calls.
//
//   #include <tile_collectives.cuh>
//   #include <user_kernel.cuh>
//   __global__ void my_kernel(tileccl::SymmWindow w, tileccl::UserArgs a) { ... }
//   TILECCL_USER_KERNEL_MAIN(my_kernel)
//
// TILECCL_USER_KERNEL_MAIN_COOPERATIVE launches with cudaLaunchCooperativeKernel:
// every CTA of the grid is then resident at once, which a kernel whose CTAs wait
// for one another (for instance one CTA per emulated rank on a single GPU) needs.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "symm_ptr.cuh"

namespace tileccl {

static constexpr int kUserMaxArgs = 16;
struct UserArgs {
  uint64_t v[kUserMaxArgs];   // device addresses, sizes, epochs: whatever the kernel expects
  int32_t n;
};

template <typename T>
__device__ __forceinline__ T* user_ptr(const UserArgs& a, int i) {
  return reinterpret_cast<T*>(a.v[i]);
}

}  // namespace tileccl

// The entry macros also define `tileccl_user_debug_read(void* record, int clear)`: the
// record of bounds violations of this object when it was compiled with
// -DTILECCL_DEBUG_CHECKS (userkernel.compile(..., debug=True)), an empty record otherwise.
#define TILECCL_USER_KERNEL_ENTRY_(KERNEL, COOPERATIVE)                                       \
  TILECCL_DEFINE_DEBUG_READER(tileccl_user_debug_read)                                        \
  extern "C" int tileccl_user_launch(const tileccl::SymmWindow* w, const uint64_t* args,      \
                                     int n_args, int grid, int block, void* stream) {         \
    tileccl::UserArgs a = {};                                                                 \
    a.n = n_args < tileccl::kUserMaxArgs ? n_args : tileccl::kUserMaxArgs;                    \
    for (int i = 0; i < a.n; ++i) a.v[i] = args[i];                                           \
    tileccl::SymmWindow win = *w;                                                             \
    if (COOPERATIVE) {                                                                        \
      void* params[2] = {&win, &a};                                                           \
      cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(KERNEL),      \
                                                  dim3(grid), dim3(block), params, 0,         \
                                                  static_cast<cudaStream_t>(stream));         \
      return static_cast<int>(e);                                                             \
    }                                                                                         \
    KERNEL<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(win, a);                    \
    return static_cast<int>(cudaGetLastError());                                              \
  }
#define TILECCL_USER_KERNEL_MAIN(KERNEL) TILECCL_USER_KERNEL_ENTRY_(KERNEL, false)
#define TILECCL_USER_KERNEL_MAIN_COOPERATIVE(KERNEL) TILECCL_USER_KERNEL_ENTRY_(KERNEL, true)
