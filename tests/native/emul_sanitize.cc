// Driver that runs the CPU emulation of the fused operators (one thread per rank,
// csrc/cpu_emul/fake_device.cc) under ThreadSanitizer / AddressSanitizer.  The emulator
// uses the same tile order, TileGroup counters, late signalling and flush-before-wait
// rules as the sm_100a kernel, with std::atomic release / acquire in place of the
// system-scope flags, so a data race or an out-of-bounds index in the protocol shows up
// here as a sanitizer report.  Built and run by tests/test_emulator_sanitizers.py:
//
//   g++ -std=c++17 -O1 -g -fsanitize=thread -I <cuda>/include emul_sanitize.cc \
//       <repo>/tileccl_b200/csrc/cpu_emul/fake_device.cc -lpthread -o emul_tsan
//
// Exit code 0 = every case matched the straight fp32 reference (and the fault cases timed
// out the way they should); sanitizer findings make the process exit non-zero by themselves.
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <string>
#include <vector>

#include "../../tileccl_b200/csrc/api.h"

namespace tileccl {
// The emulator only needs the error-message hooks of runtime/errors.cc.
static thread_local std::string g_msg;
void set_last_error(const std::string& msg) { g_msg = msg; }
const std::string& last_error() { return g_msg; }
}  // namespace tileccl

namespace {

uint32_t g_seed = 12345;
float frand() {
  g_seed = g_seed * 1664525u + 1013904223u;
  return static_cast<float>((g_seed >> 8) & 0xFFFF) / 32768.0f - 1.0f;
}

int check(const char* what, const std::vector<float>& got, const std::vector<float>& want) {
  double worst = 0;
  for (size_t i = 0; i < got.size(); ++i) worst = std::fmax(worst, std::fabs(got[i] - want[i]));
  if (worst > 1e-3) {
    std::fprintf(stderr, "%s: max abs error %g\n", what, worst);
    return 1;
  }
  return 0;
}

// C[r-th block of rows] = A_r @ B_r, gathered on every rank.
int run_allgather(int ws, int M, int N, int K, int bm, int bn, int gm, int fault_rank, int fault,
                  int expect_code) {
  const int mloc = M / ws;
  std::vector<float> A(static_cast<size_t>(ws) * mloc * K), B(static_cast<size_t>(ws) * K * N);
  std::vector<float> C(static_cast<size_t>(ws) * M * N, 0.f), want(static_cast<size_t>(M) * N);
  for (auto& x : A) x = frand();
  for (auto& x : B) x = frand();
  for (int r = 0; r < ws; ++r)
    for (int i = 0; i < mloc; ++i)
      for (int j = 0; j < N; ++j) {
        double acc = 0;
        for (int k = 0; k < K; ++k)
          acc += static_cast<double>(A[(static_cast<size_t>(r) * mloc + i) * K + k]) *
                 B[(static_cast<size_t>(r) * K + k) * N + j];
        want[(static_cast<size_t>(r) * mloc + i) * N + j] = static_cast<float>(acc);
      }
  int32_t status[6] = {0, 0, 0, 0, 0, 0};
  const int rc = tccl_emul_gemm_allgather(ws, M, N, K, A.data(), B.data(), C.data(), bm, bn, gm,
                                          fault_rank, fault, 20, fault ? 150 : 20000, status);
  if (rc != 0) {
    std::fprintf(stderr, "allgather ws=%d: rc=%d (%s)\n", ws, rc, tileccl::last_error().c_str());
    return 1;
  }
  if (status[0] != expect_code) {
    std::fprintf(stderr, "allgather ws=%d fault=%d: status %d, expected %d\n", ws, fault, status[0],
                 expect_code);
    return 1;
  }
  if (expect_code != 0) return 0;
  int bad = 0;
  for (int r = 0; r < ws; ++r) {
    std::vector<float> got(C.begin() + static_cast<size_t>(r) * M * N,
                           C.begin() + static_cast<size_t>(r + 1) * M * N);
    bad += check("allgather", got, want);
  }
  return bad;
}

// C_r = rows r of sum over ranks of A_s @ B_s (K split over ranks).
int run_reducescatter(int ws, int M, int N, int K, int bm, int bn, int gm, int own_lag, int delay,
                      int fault_rank, int fault, int expect_code) {
  const int kloc = K / ws, mloc = M / ws;
  std::vector<float> A(static_cast<size_t>(ws) * M * kloc), B(static_cast<size_t>(ws) * kloc * N);
  std::vector<float> C(static_cast<size_t>(ws) * mloc * N, 0.f), want(static_cast<size_t>(M) * N);
  for (auto& x : A) x = frand();
  for (auto& x : B) x = frand();
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double acc = 0;
      for (int s = 0; s < ws; ++s)
        for (int k = 0; k < kloc; ++k)
          acc += static_cast<double>(A[(static_cast<size_t>(s) * M + i) * kloc + k]) *
                 B[(static_cast<size_t>(s) * kloc + k) * N + j];
      want[static_cast<size_t>(i) * N + j] = static_cast<float>(acc);
    }
  int32_t status[6] = {0, 0, 0, 0, 0, 0};
  const int rc = tccl_emul_gemm_reducescatter_ex(ws, M, N, K, A.data(), B.data(), C.data(), bm, bn,
                                                 gm, own_lag, delay, 1, fault_rank, fault, 20,
                                                 fault ? 150 : 20000, status);
  if (rc != 0) {
    std::fprintf(stderr, "reducescatter ws=%d: rc=%d (%s)\n", ws, rc,
                 tileccl::last_error().c_str());
    return 1;
  }
  if (status[0] != expect_code) {
    std::fprintf(stderr, "reducescatter ws=%d fault=%d: status %d, expected %d\n", ws, fault,
                 status[0], expect_code);
    return 1;
  }
  if (expect_code != 0) return 0;
  return check("reducescatter", C, want);
}

}  // namespace

int main() {
  int bad = 0;
  for (int ws : {2, 4, 8}) {
    bad += run_allgather(ws, 64 * ws, 96, 40, 16, 32, 1, -1, 0, 0);
    bad += run_allgather(ws, 32 * ws, 64, 24, 16, 32, 2, -1, 0, 0);
    for (int lag : {0, 2})
      for (int delay : {0, 1, 2}) bad += run_reducescatter(ws, 32 * ws, 64, 8 * ws, 16, 32, 1, lag,
                                                           delay, -1, 0, 0);
  }
  // host-side faults: a rank that moves data but never signals (1), one that never runs (3);
  // the others must give up with the signal time-out code (2), not hang
  bad += run_allgather(4, 128, 64, 16, 16, 32, 1, 2, 1, 2);
  bad += run_allgather(2, 64, 64, 16, 16, 32, 1, 1, 3, 2);
  bad += run_reducescatter(4, 128, 64, 32, 16, 32, 1, 0, 1, 3, 1, 2);
  std::printf(bad ? "emul_sanitize: %d case(s) FAILED\n" : "emul_sanitize: all cases ok\n", bad);
  return bad ? 1 : 0;
}
