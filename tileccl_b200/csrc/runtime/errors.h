// Error plumbing shared by the C ABI: a thread-local message and helpers that
// turn CUDA runtime / driver statuses into "return non-zero + message".
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <sstream>
#include <string>

#include "driver_api.h"

namespace tileccl {

void set_last_error(const std::string& msg);
const std::string& last_error();

enum ReturnCode : int {
  kOk = 0,
  kErrInvalid = 1,      // bad argument
  kErrCuda = 2,         // CUDA runtime / driver call failed
  kErrUnsupported = 3,  // no driver / feature missing on this machine
  kErrSystem = 4,       // socket / OS failure
  kErrTimeout = 5,
};

inline int fail(int code, const std::string& msg) {
  set_last_error(msg);
  return code;
}

}  // namespace tileccl

#define TCCL_CHECK_ARG(cond, msg)                                              \
  do {                                                                         \
    if (!(cond)) {                                                             \
      std::ostringstream tccl_os;                                              \
      tccl_os << msg;                                                          \
      return ::tileccl::fail(::tileccl::kErrInvalid, tccl_os.str());           \
    }                                                                          \
  } while (0)

#define TCCL_CHECK_CUDA(expr)                                                  \
  do {                                                                         \
    cudaError_t tccl_e = (expr);                                               \
    if (tccl_e != cudaSuccess) {                                               \
      return ::tileccl::fail(::tileccl::kErrCuda,                              \
                             std::string(#expr) + ": " + cudaGetErrorString(tccl_e)); \
    }                                                                          \
  } while (0)

#define TCCL_CHECK_CU(expr)                                                    \
  do {                                                                         \
    CUresult tccl_r = (expr);                                                  \
    if (tccl_r != CUDA_SUCCESS) {                                              \
      return ::tileccl::fail(::tileccl::kErrCuda,                              \
                             std::string(#expr) + ": " +                       \
                                 ::tileccl::driver_error_string(tccl_r));      \
    }                                                                          \
  } while (0)

#define TCCL_REQUIRE_DRIVER()                                                  \
  do {                                                                         \
    if (!::tileccl::driver().ok)                                               \
      return ::tileccl::fail(::tileccl::kErrUnsupported,                       \
                             "CUDA driver not available: " + ::tileccl::driver().error); \
  } while (0)
