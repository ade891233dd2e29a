// CPU emulation of the multi-rank fused operators: one std::thread per rank, a
// "symmetric heap" that is plain host memory visible to all threads, and
// std::atomic counters with release / acquire ordering standing in for the
// system-scope flags of the GPU kernels.  Each rank walks the SAME tile order as
// the sm_100a kernel (plan/tile_order.h), computes its tiles in fp32, pushes them
// to the peers, signals TileGroup counters and waits for the peers' signals with
// a bounded wait.
//
// Two uses: (1) a GPU-free oracle for GEMM + all-gather and GEMM ->
// reduce-scatter semantics and for the signalling protocol; (2) host-side fault
// injection: a rank that never signals, signals too little, or never starts must
// make the other ranks time out and report, never hang.
#include <atomic>
#include <chrono>
#include <cstring>
#include <deque>
#include <memory>
#include <thread>
#include <utility>
#include <vector>

#include "../api.h"
#include "../plan/tile_order.h"
#include "../runtime/errors.h"

namespace tileccl {
namespace {

enum Fault : int {
  kFaultNone = 0,
  kFaultNoSignal = 1,    // moves data but never signals
  kFaultShortSignal = 2, // signals every other tile only (a stale / incomplete epoch)
  kFaultAbsent = 3,      // the rank never runs
  kFaultLate = 4,        // the rank starts after `fault_delay_ms`
};

struct Counters {
  // counters[dest][src * groups + g]
  std::vector<std::unique_ptr<std::atomic<uint32_t>[]>> per_rank;
  int groups = 0, ws = 0;
  void init(int world, int n_groups) {
    ws = world;
    groups = n_groups;
    per_rank.resize(world);
    for (auto& p : per_rank) {
      p.reset(new std::atomic<uint32_t>[static_cast<size_t>(world) * n_groups]);
      for (int i = 0; i < world * n_groups; ++i) p[i].store(0, std::memory_order_relaxed);
    }
  }
  std::atomic<uint32_t>& at(int dest, int src, int g) { return per_rank[dest][src * groups + g]; }
};

// Bounded acquire-wait: false on time-out (`*seen` = last value).
bool wait_ge(std::atomic<uint32_t>& c, uint32_t target, int timeout_ms, uint32_t* seen) {
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  for (int spin = 0;; ++spin) {
    const uint32_t v = c.load(std::memory_order_acquire);
    if (static_cast<int32_t>(v - target) >= 0) return true;
    if ((spin & 0x3ff) == 0x3ff) {
      if (std::chrono::steady_clock::now() > deadline) {
        *seen = v;
        return false;
      }
      std::this_thread::yield();
    }
  }
}

// out[rows x cols] (ld_out) = A[rows x K] (lda) @ B[K x cols] (ldb), fp32
void tile_gemm(const float* A, int64_t lda, const float* B, int64_t ldb, float* out, int64_t ldo,
               int rows, int cols, int K) {
  for (int i = 0; i < rows; ++i) {
    float* o = out + i * ldo;
    for (int j = 0; j < cols; ++j) o[j] = 0.f;
    for (int k = 0; k < K; ++k) {
      const float a = A[i * lda + k];
      const float* b = B + k * ldb;
      for (int j = 0; j < cols; ++j) o[j] += a * b[j];
    }
  }
}

struct Status {
  std::atomic<int> code{0};
  int where = 0, rank = -1, item = -1;
  uint32_t expected = 0, observed = 0;
  void report(int c, int w, int r, int it, uint32_t exp, uint32_t obs) {
    int zero = 0;
    if (code.compare_exchange_strong(zero, c)) {
      where = w; rank = r; item = it; expected = exp; observed = obs;
    }
  }
};

inline int imin(int a, int b) { return a < b ? a : b; }

}  // namespace
}  // namespace tileccl

using namespace tileccl;

// status_out: int32[6] = {code (0 ok, 2 signal time-out), where, rank, item, expected, observed}
extern "C" int tccl_emul_gemm_allgather(int32_t world_size, int32_t M, int32_t N, int32_t K,
                                        const float* A_all, const float* B_all, float* C_all,
                                        int32_t block_m, int32_t block_n, int32_t group_m_tiles,
                                        int32_t fault_rank, int32_t fault_kind,
                                        int32_t fault_delay_ms, int32_t timeout_ms,
                                        int32_t* status_out) {
  TCCL_CHECK_ARG(world_size >= 1 && world_size <= 64, "world_size must be 1..64");
  TCCL_CHECK_ARG(M > 0 && N > 0 && K > 0 && M % world_size == 0, "bad problem shape");
  TCCL_CHECK_ARG(block_m > 0 && block_n > 0 && group_m_tiles > 0, "bad tile shape");
  TCCL_CHECK_ARG(A_all && B_all && C_all && status_out, "null argument");
  const int ws = world_size, mloc = M / ws;
  const int m_tiles = (mloc + block_m - 1) / block_m, n_tiles = (N + block_n - 1) / block_n;
  const int groups = (m_tiles + group_m_tiles - 1) / group_m_tiles;
  Counters sig;
  sig.init(ws, groups);
  Status status;

  auto body = [&](int rank) {
    if (rank == fault_rank && fault_kind == kFaultAbsent) return;
    if (rank == fault_rank && fault_kind == kFaultLate)
      std::this_thread::sleep_for(std::chrono::milliseconds(fault_delay_ms));
    const float* A = A_all + static_cast<int64_t>(rank) * mloc * K;
    const float* B = B_all + static_cast<int64_t>(rank) * K * N;
    const TileOrderShape shape{m_tiles, n_tiles, 1, rank, ws, 0};
    std::vector<float> tile(static_cast<size_t>(block_m) * block_n);
    for (int t = 0; t < tile_order_count(shape); ++t) {
      const TileOrderEntry e = tile_order_decode(shape, t);
      const int r0 = e.lm * block_m, c0 = e.ln * block_n;
      const int rows = imin(block_m, mloc - r0), cols = imin(block_n, N - c0);
      tile_gemm(A + static_cast<int64_t>(r0) * K, K, B + c0, N, tile.data(), block_n, rows, cols, K);
      for (int d = 0; d < ws; ++d) {  // push to every rank's C (own copy included)
        float* C = C_all + static_cast<int64_t>(d) * M * N;
        for (int i = 0; i < rows; ++i)
          std::memcpy(C + (static_cast<int64_t>(rank) * mloc + r0 + i) * N + c0,
                      tile.data() + static_cast<int64_t>(i) * block_n, sizeof(float) * cols);
      }
      bool signal = true;
      if (rank == fault_rank && fault_kind == kFaultNoSignal) signal = false;
      if (rank == fault_rank && fault_kind == kFaultShortSignal && (t & 1)) signal = false;
      if (signal) {
        const int g = e.lm / group_m_tiles;
        for (int d = 0; d < ws; ++d)
          if (d != rank) sig.at(d, rank, g).fetch_add(1, std::memory_order_release);
      }
    }
    // consumer side: every peer's TileGroups must have arrived
    for (int src = 0; src < ws; ++src) {
      if (src == rank) continue;
      for (int g = 0; g < groups; ++g) {
        const int rows_in_group = imin(group_m_tiles, m_tiles - g * group_m_tiles);
        const uint32_t target = static_cast<uint32_t>(rows_in_group * n_tiles);
        uint32_t seen = 0;
        if (!wait_ge(sig.at(rank, src, g), target, timeout_ms, &seen)) {
          status.report(2, 30, rank, src * groups + g, target, seen);
          return;
        }
      }
    }
  };
  std::vector<std::thread> threads;
  for (int r = 0; r < ws; ++r) threads.emplace_back(body, r);
  for (auto& th : threads) th.join();
  status_out[0] = status.code.load();
  status_out[1] = status.where;
  status_out[2] = status.rank;
  status_out[3] = status.item;
  status_out[4] = static_cast<int32_t>(status.expected);
  status_out[5] = static_cast<int32_t>(status.observed);
  return kOk;
}

extern "C" int tccl_emul_gemm_reducescatter_ex(int32_t world_size, int32_t M, int32_t N,
                                               int32_t K_total, const float* A_all,
                                               const float* B_all, float* C_all, int32_t block_m,
                                               int32_t block_n, int32_t group_m_tiles,
                                               int32_t own_lag, int32_t signal_delay_tiles,
                                               int32_t flush_before_wait, int32_t fault_rank,
                                               int32_t fault_kind, int32_t fault_delay_ms,
                                               int32_t timeout_ms, int32_t* status_out);

// A_all: [ws][M][K/ws], B_all: [ws][K/ws][N], C_all: [ws][M/ws][N]
extern "C" int tccl_emul_gemm_reducescatter(int32_t world_size, int32_t M, int32_t N,
                                            int32_t K_total, const float* A_all,
                                            const float* B_all, float* C_all, int32_t block_m,
                                            int32_t block_n, int32_t group_m_tiles,
                                            int32_t fault_rank, int32_t fault_kind,
                                            int32_t fault_delay_ms, int32_t timeout_ms,
                                            int32_t* status_out) {
  return tccl_emul_gemm_reducescatter_ex(world_size, M, N, K_total, A_all, B_all, C_all, block_m,
                                         block_n, group_m_tiles, 0, 0, 1, fault_rank, fault_kind,
                                         fault_delay_ms, timeout_ms, status_out);
}

// Same with the ranks' own tile rows trailing the remote rounds by `own_lag` rounds
// (plan/tile_order.h): every rank is one thread that walks its tile order and blocks at its
// own tiles, so this also exercises the schedule's freedom from deadlock.
// `signal_delay_tiles` models the kernel's late signalling: the signal of a tile is sent
// only when that many later tiles have been finished (the data of a bulk store must have
// landed first); `flush_before_wait` sends everything still held before a rank blocks at
// one of its own tiles.  Without the flush, ranks that all hold the signals their peers are
// waiting for stop each other.
extern "C" int tccl_emul_gemm_reducescatter_ex(int32_t world_size, int32_t M, int32_t N,
                                               int32_t K_total, const float* A_all,
                                               const float* B_all, float* C_all, int32_t block_m,
                                               int32_t block_n, int32_t group_m_tiles,
                                               int32_t own_lag, int32_t signal_delay_tiles,
                                               int32_t flush_before_wait, int32_t fault_rank,
                                               int32_t fault_kind, int32_t fault_delay_ms,
                                               int32_t timeout_ms, int32_t* status_out) {
  TCCL_CHECK_ARG(own_lag >= 0 && signal_delay_tiles >= 0, "own_lag and signal_delay_tiles must be >= 0");
  TCCL_CHECK_ARG(world_size >= 1 && world_size <= 64, "world_size must be 1..64");
  TCCL_CHECK_ARG(M > 0 && N > 0 && K_total > 0 && M % world_size == 0 && K_total % world_size == 0,
                 "bad problem shape");
  TCCL_CHECK_ARG(block_m > 0 && block_n > 0 && group_m_tiles > 0, "bad tile shape");
  TCCL_CHECK_ARG(A_all && B_all && C_all && status_out, "null argument");
  const int ws = world_size, mloc = M / ws, kloc = K_total / ws;
  const int m_tiles = (mloc + block_m - 1) / block_m, n_tiles = (N + block_n - 1) / block_n;
  const int groups = (m_tiles + group_m_tiles - 1) / group_m_tiles;
  Counters sig;          // sig.at(owner, 0, g): partial tiles of group g that reached the owner
  sig.init(ws, groups);
  Status status;
  // staging[owner][src][mloc][N]: partial sums pushed by `src` for the owner's rows
  std::vector<std::vector<float>> staging(ws);
  for (auto& s : staging) s.assign(static_cast<size_t>(ws) * mloc * N, 0.f);

  auto body = [&](int rank) {
    if (rank == fault_rank && fault_kind == kFaultAbsent) return;
    if (rank == fault_rank && fault_kind == kFaultLate)
      std::this_thread::sleep_for(std::chrono::milliseconds(fault_delay_ms));
    const float* A = A_all + static_cast<int64_t>(rank) * M * kloc;
    const float* B = B_all + static_cast<int64_t>(rank) * kloc * N;
    float* C = C_all + static_cast<int64_t>(rank) * mloc * N;
    const TileOrderShape shape{m_tiles, n_tiles, ws, rank, ws, 0, own_lag};
    std::vector<float> tile(static_cast<size_t>(block_m) * block_n);
    // signals not sent yet: one entry per finished tile, (owner, group) or owner = -1 for none
    std::deque<std::pair<int, int>> held;
    auto release = [&](size_t keep) {
      while (held.size() > keep) {
        const auto s = held.front();
        held.pop_front();
        if (s.first >= 0) sig.at(s.first, 0, s.second).fetch_add(1, std::memory_order_release);
      }
    };
    for (int t = 0; t < tile_order_count(shape); ++t) {
      const TileOrderEntry e = tile_order_decode(shape, t);
      const int r0 = e.lm * block_m, c0 = e.ln * block_n;
      const int rows = imin(block_m, mloc - r0), cols = imin(block_n, N - c0);
      const int g = e.lm / group_m_tiles;
      tile_gemm(A + (static_cast<int64_t>(e.owner) * mloc + r0) * kloc, kloc, B + c0, N, tile.data(),
                block_n, rows, cols, kloc);
      if (e.owner != rank) {
        float* slot = staging[e.owner].data() + static_cast<int64_t>(rank) * mloc * N;
        for (int i = 0; i < rows; ++i)
          std::memcpy(slot + static_cast<int64_t>(r0 + i) * N + c0,
                      tile.data() + static_cast<int64_t>(i) * block_n, sizeof(float) * cols);
        bool signal = true;
        if (rank == fault_rank && fault_kind == kFaultNoSignal) signal = false;
        if (rank == fault_rank && fault_kind == kFaultShortSignal && (t & 1)) signal = false;
        held.emplace_back(signal ? e.owner : -1, g);
        release(static_cast<size_t>(signal_delay_tiles));
      } else {
        // own tile: wait for the peers' partials of this TileGroup, add them in rank order
        const int rows_in_group = imin(group_m_tiles, m_tiles - g * group_m_tiles);
        const uint32_t target = static_cast<uint32_t>((ws - 1) * rows_in_group * n_tiles);
        uint32_t seen = 0;
        if (ws > 1 && flush_before_wait &&
            sig.at(rank, 0, g).load(std::memory_order_acquire) < target)
          release(0);
        if (ws > 1 && !wait_ge(sig.at(rank, 0, g), target, timeout_ms, &seen)) {
          status.report(2, 40, rank, g, target, seen);
          return;
        }
        for (int src = 0; src < ws; ++src) {
          if (src == rank) continue;
          const float* slot = staging[rank].data() + static_cast<int64_t>(src) * mloc * N;
          for (int i = 0; i < rows; ++i)
            for (int j = 0; j < cols; ++j)
              tile[static_cast<int64_t>(i) * block_n + j] += slot[static_cast<int64_t>(r0 + i) * N + c0 + j];
        }
        for (int i = 0; i < rows; ++i)
          std::memcpy(C + static_cast<int64_t>(r0 + i) * N + c0,
                      tile.data() + static_cast<int64_t>(i) * block_n, sizeof(float) * cols);
        held.emplace_back(-1, g);
        release(static_cast<size_t>(signal_delay_tiles));
      }
    }
    release(0);
  };
  std::vector<std::thread> threads;
  for (int r = 0; r < ws; ++r) threads.emplace_back(body, r);
  for (auto& th : threads) th.join();
  status_out[0] = status.code.load();
  status_out[1] = status.where;
  status_out[2] = status.rank;
  status_out[3] = status.item;
  status_out[4] = static_cast<int32_t>(status.expected);
  status_out[5] = static_cast<int32_t>(status.observed);
  return kOk;
}

// Tile order of one rank as (owner, lm, ln) triples, for tests of the schedule.
extern "C" int tccl_plan_tile_order_ex(int32_t m_tiles_local, int32_t n_tiles_local,
                                       int32_t owners, int32_t rank, int32_t world_size,
                                       int32_t rot_m_tiles, int32_t own_lag, int32_t* out,
                                       int32_t capacity);

extern "C" int tccl_plan_tile_order(int32_t m_tiles_local, int32_t n_tiles_local, int32_t owners,
                                    int32_t rank, int32_t world_size, int32_t rot_m_tiles,
                                    int32_t* out, int32_t capacity) {
  return tccl_plan_tile_order_ex(m_tiles_local, n_tiles_local, owners, rank, world_size,
                                 rot_m_tiles, 0, out, capacity);
}

extern "C" int tccl_plan_tile_order_ex(int32_t m_tiles_local, int32_t n_tiles_local,
                                       int32_t owners, int32_t rank, int32_t world_size,
                                       int32_t rot_m_tiles, int32_t own_lag, int32_t* out,
                                       int32_t capacity) {
  TCCL_CHECK_ARG(m_tiles_local > 0 && n_tiles_local > 0 && owners >= 1 && out != nullptr, "bad argument");
  TCCL_CHECK_ARG(own_lag >= 0, "own_lag must be >= 0");
  const TileOrderShape shape{m_tiles_local, n_tiles_local, owners, rank, world_size, rot_m_tiles,
                             own_lag};
  const int n = tile_order_count(shape);
  TCCL_CHECK_ARG(capacity >= n, "output too small");
  for (int t = 0; t < n; ++t) {
    const TileOrderEntry e = tile_order_decode(shape, t);
    out[3 * t] = e.owner;
    out[3 * t + 1] = e.lm;
    out[3 * t + 2] = e.ln;
  }
  return kOk;
}
