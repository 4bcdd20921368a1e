// Launch-shape selection: rows per block, tree threads, rows per lane, tree chunks,
// staging.  Takes the place of the reference's auto-scheduler and exhaustive
// auto-tuner (src/mlir/GPUAutoSchedule.cpp:318-472 loop-nest construction, :525-971
// timed search over rowsPerTB x treeThreads x representation x unroll/interleave,
// shared-memory guard src/test/GPUBenchmarkUtils.h:387-402): the kernel family is
// fixed, so selection is a closed-form choice under the shared-memory budget whose
// constants come from profiling on B200, not a compile-and-time loop.
#pragma once
#include "../../include/tbk.h"

#include <cstdint>
#include <string>

namespace tb {

struct ForestShape {
  int32_t num_features;
  int32_t num_classes;
  int64_t num_groups;
  uint64_t max_group_bytes;
  int32_t lut_bytes;
  int32_t representation;
  int32_t tile_size;
};

struct LaunchPlan {
  int32_t row_warps = 1;     // warps along the row dimension of a block
  int32_t tree_threads = 1;  // warps sharing one row tile (1, 2, 4, 8 or 16)
  int32_t rows_per_lane = 1; // rows a lane walks in lock-step (1 or 2)
  int32_t chunks = 1;        // grid.y
  int32_t groups_per_chunk = 1;
  int32_t staged = 0;        // tree groups staged through shared memory
  int32_t cache_rows = 1;    // row tile transposed into shared memory
  int32_t class_regs = 0;    // multiclass: class sums in registers (no shared-memory class table)
  uint32_t stage_bytes = 0;
  int32_t smem_bytes = 0;
  int32_t threads = 32;
  int64_t grid_x = 1;
};

// Shared-memory bytes a block needs for the given shape.
int64_t smem_needed(const ForestShape &fs, const LaunchPlan &p);

// Fills `plan`; returns an empty string on success or the reason no launch shape fits.
// partial: the launch writes per-class partial sums (tree-sharded use) instead of predictions.
std::string select_launch(const ForestShape &fs, const tbk_schedule &user, int64_t n_rows,
                          int32_t smem_limit, int32_t num_sms, bool leaf_ids, LaunchPlan *plan,
                          bool partial = false);

} // namespace tb
