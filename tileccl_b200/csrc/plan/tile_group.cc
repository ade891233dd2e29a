// TileGroup planner (host, no CUDA).
//
// A TileGroup is a band of consecutive tile rows of the GEMM output: contiguous
// memory, so it can be handed to a peer as one transfer, and it completes in
// order under a row-band-major tile schedule.  Two rules shape the groups
// (same policy as the reference planner, tileccl_v2/tile_group.py:87-153):
//   P0  a group holds at least ceil(tau_min_bytes / tile_bytes) tiles, so that one
//       group is large enough to saturate the link;
//   P1  group boundaries fall on multiples of `group_m` tile rows (the
//       rasterisation wave of the GEMM), the ragged tail joins the last group.
// More than `max_groups` groups are merged pairwise-or-more until they fit.
// Groups can then be cut at row-ownership boundaries so that none spans two
// owners of a reduce-scatter.
//
// This is the single definition of the policy: the Python planning API
// (tileccl_b200/planning/tile_group.py) calls it through the C ABI.
#include <algorithm>
#include <cstdint>
#include <vector>

#include "../api.h"
#include "../runtime/errors.h"

namespace tileccl {
namespace {

struct Group {
  int64_t row_start, row_end, tiles;
};

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

std::vector<Group> plan_groups(int64_t M, int64_t N, int64_t tile_bytes, int64_t target_tiles,
                               int32_t max_groups, int32_t block_m, int32_t block_n,
                               int32_t group_m, int64_t tau_min_bytes) {
  const int64_t tile_rows = ceil_div(M, block_m);
  const int64_t tile_cols = ceil_div(N, block_n);
  const int64_t p0 = std::max<int64_t>(1, ceil_div(tau_min_bytes, tile_bytes));
  const int64_t want = std::max<int64_t>(p0, target_tiles > 0 ? target_tiles : p0);

  std::vector<Group> groups;
  int64_t open_row = 0;   // first tile row of the group being filled
  int64_t held = 0;       // tiles collected so far
  for (int64_t wave = 0; wave < tile_rows; wave += group_m) {
    const int64_t wave_end = std::min<int64_t>(wave + group_m, tile_rows);
    held += (wave_end - wave) * tile_cols;
    if (held >= want) {
      groups.push_back({open_row * block_m, wave_end * block_m, held});
      open_row = wave_end;
      held = 0;
    }
  }
  if (held > 0) {
    if (groups.empty()) groups.push_back({0, M, held});
    else {
      groups.back().row_end = M;
      groups.back().tiles += held;
    }
  }
  if (static_cast<int64_t>(groups.size()) > max_groups) {
    const int64_t fold = ceil_div(static_cast<int64_t>(groups.size()), max_groups);
    std::vector<Group> merged;
    for (size_t i = 0; i < groups.size(); i += fold) {
      Group g = groups[i];
      for (size_t j = i + 1; j < std::min(groups.size(), i + fold); ++j) {
        g.row_end = groups[j].row_end;
        g.tiles += groups[j].tiles;
      }
      g.row_end = std::min(g.row_end, M);
      merged.push_back(g);
    }
    groups.swap(merged);
  }
  return groups;
}

std::vector<Group> cut_at(const std::vector<Group>& groups, int64_t M, int64_t N,
                          std::vector<int64_t> cuts, int32_t block_m, int32_t block_n) {
  const int64_t tile_cols = ceil_div(N, block_n);
  cuts.erase(std::remove_if(cuts.begin(), cuts.end(), [M](int64_t c) { return c <= 0 || c >= M; }),
             cuts.end());
  cuts.push_back(M);
  std::sort(cuts.begin(), cuts.end());
  cuts.erase(std::unique(cuts.begin(), cuts.end()), cuts.end());
  std::vector<Group> out;
  for (const Group& g : groups) {
    const int64_t end = std::min(g.row_end, M);
    int64_t at = g.row_start;
    while (at < end) {
      const int64_t next_cut = *std::upper_bound(cuts.begin(), cuts.end(), at);
      const int64_t stop = std::min(end, next_cut);
      out.push_back({at, stop, ceil_div(stop - at, block_m) * tile_cols});
      at = stop;
    }
  }
  return out;
}

}  // namespace
}  // namespace tileccl

using namespace tileccl;

extern "C" int tccl_plan_tile_groups(int64_t M, int64_t N, int64_t tile_bytes,
                                     int64_t target_group_tiles, int32_t max_groups,
                                     int32_t block_m, int32_t block_n, int32_t group_m,
                                     int64_t tau_min_bytes, const int64_t* row_boundaries,
                                     int32_t n_boundaries, int64_t* groups_out, int32_t capacity,
                                     int32_t* n_groups_out) {
  TCCL_CHECK_ARG(M > 0 && N > 0, "M and N must be positive");
  TCCL_CHECK_ARG(tile_bytes > 0, "tile_bytes must be positive");
  TCCL_CHECK_ARG(block_m > 0 && block_n > 0 && group_m > 0,
                 "block_m, block_n, and group_m must be positive");
  TCCL_CHECK_ARG(max_groups > 0, "max_groups must be positive");
  TCCL_CHECK_ARG(groups_out != nullptr && n_groups_out != nullptr, "null output");
  std::vector<Group> groups =
      plan_groups(M, N, tile_bytes, target_group_tiles, max_groups, block_m, block_n, group_m,
                  tau_min_bytes);
  if (n_boundaries > 0 && row_boundaries != nullptr)
    groups = cut_at(groups, M, N, std::vector<int64_t>(row_boundaries, row_boundaries + n_boundaries),
                    block_m, block_n);
  TCCL_CHECK_ARG(static_cast<int64_t>(groups.size()) <= capacity,
                 "output buffer too small for " << groups.size() << " groups");
  for (size_t i = 0; i < groups.size(); ++i) {
    groups_out[3 * i + 0] = groups[i].row_start;
    groups_out[3 * i + 1] = groups[i].row_end;
    groups_out[3 * i + 2] = groups[i].tiles;
  }
  *n_groups_out = static_cast<int32_t>(groups.size());
  return kOk;
}

// tile id (in the group_m-swizzled rasterisation: within a wave of group_m tile
// rows, consecutive ids walk down the rows first) -> index of the group that
// holds the tile's first row.  Tiles outside every group map to 0.
extern "C" int tccl_plan_group_table(int64_t M, int64_t N, const int64_t* groups, int32_t n_groups,
                                     int32_t block_m, int32_t block_n, int32_t group_m,
                                     int32_t* table_out, int64_t table_len) {
  TCCL_CHECK_ARG(M > 0 && N > 0 && block_m > 0 && block_n > 0 && group_m > 0, "bad shape");
  TCCL_CHECK_ARG(groups != nullptr && table_out != nullptr && n_groups >= 0, "null argument");
  const int64_t tile_rows = ceil_div(M, block_m);
  const int64_t tile_cols = ceil_div(N, block_n);
  TCCL_CHECK_ARG(table_len == tile_rows * tile_cols, "table length must equal the tile count");
  // group id per tile row (first match wins, as a linear scan would give)
  std::vector<int32_t> row_gid(tile_rows, 0);
  for (int64_t tr = 0; tr < tile_rows; ++tr) {
    const int64_t row = tr * block_m;
    for (int32_t g = 0; g < n_groups; ++g) {
      if (groups[3 * g] <= row && row < groups[3 * g + 1]) {
        row_gid[tr] = g;
        break;
      }
    }
  }
  const int64_t per_wave = static_cast<int64_t>(group_m) * tile_cols;
  for (int64_t id = 0; id < table_len; ++id) {
    const int64_t wave = id / per_wave;
    const int64_t first_row = wave * group_m;
    const int64_t rows_here = std::min<int64_t>(tile_rows - first_row, group_m);
    const int64_t tr = first_row + (id % per_wave) % rows_here;
    table_out[id] = row_gid[tr];
  }
  return kOk;
}
