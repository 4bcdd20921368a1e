#include "schedule.h"

#include <algorithm>

namespace tb {

static int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

int64_t smem_needed(const ForestShape &fs, const LaunchPlan &p) {
  const int64_t rt = 32 * p.rows_per_lane;
  int64_t bytes = align_up(16 + fs.lut_bytes, 128);
  if (p.staged) bytes += 2 * (int64_t)p.stage_bytes;
  if (p.cache_rows) bytes += (int64_t)p.row_warps * (fs.num_features + 1) * rt * 4;
  const int64_t warps = (int64_t)p.row_warps * p.tree_threads;
  if (fs.num_classes > 0 && !p.class_regs)
    bytes += warps * fs.num_classes * rt * 4;
  else if (p.tree_threads > 1)
    bytes += warps * rt * 4;
  return bytes;
}

static int floor_pow2(int v) {
  int p = 1;
  while (p * 2 <= v) p *= 2;
  return p;
}

std::string select_launch(const ForestShape &fs, const tbk_schedule &user, int64_t n_rows,
                          int32_t smem_limit, int32_t num_sms, bool leaf_ids, LaunchPlan *out, bool partial) {
  (void)leaf_ids;
  if (n_rows <= 0) n_rows = 1;
  if (num_sms <= 0) num_sms = 148;
  if (smem_limit <= 0) smem_limit = 227 * 1024;
  const int max_warps = 32;
  LaunchPlan best;
  bool have = false;

  const uint32_t stage_bytes = (uint32_t)align_up((int64_t)fs.max_group_bytes, 128);
  // staging pays when two stages leave at least ~40% of shared memory to the rows
  const bool can_stage = 2 * (int64_t)stage_bytes <= (int64_t)smem_limit * 6 / 10 && stage_bytes < (1u << 20);
  const bool want_stage = user.cache_trees == 2 ? false : can_stage;
  if (user.cache_trees == 1 && !can_stage)
    return "tree groups of this forest do not fit the shared-memory stages (cache_trees = 1)";

  int rpl_lo = 1, rpl_hi = 1;
  if (user.rows_per_thread >= 2) rpl_lo = rpl_hi = 2;
  else if (user.rows_per_thread == 1) rpl_lo = rpl_hi = 1;

  for (int rpl = rpl_lo; rpl <= rpl_hi && !have; ++rpl) {
    const int64_t rt = 32 * rpl;
    const int64_t row_tiles = (n_rows + rt - 1) / rt;
    // tree threads: as few as keep every SM busy with full blocks
    int tt_wanted = 1;
    if (user.tree_threads > 0) {
      tt_wanted = std::min(16, floor_pow2(user.tree_threads));
    } else if (row_tiles < (int64_t)num_sms * max_warps) {
      const int64_t tiles_per_block = std::max<int64_t>(1, row_tiles / num_sms);
      tt_wanted = std::min<int64_t>(16, floor_pow2((int)std::max<int64_t>(1, max_warps / tiles_per_block)));
    }
    for (int cached = 1; cached >= 0 && !have; --cached) {
      if (!cached && rpl != 1) continue;
      for (int tt = tt_wanted; tt <= 16 && !have; tt *= 2) {
        LaunchPlan p;
        p.rows_per_lane = rpl;
        p.tree_threads = tt;
        p.staged = want_stage;
        p.stage_bytes = want_stage ? stage_bytes : 0;
        p.cache_rows = cached;
        // class sums can stay in registers when one warp walks all trees of its rows and
        // the launch needs no tree chunks (a batch that fills the GPU twice over anyway)
        p.class_regs = fs.num_classes > 0 && tt == 1 && !partial && user.tree_chunks <= 1 &&
                       row_tiles >= 2 * (int64_t)num_sms * max_warps;
        int rw_hi = max_warps / tt;
        if (user.rows_per_block > 0) rw_hi = std::max(1, std::min<int>(rw_hi, user.rows_per_block / (int)rt));
        rw_hi = (int)std::min<int64_t>(rw_hi, row_tiles);
        for (int rw = rw_hi; rw >= 1; --rw) {
          p.row_warps = rw;
          if (smem_needed(fs, p) <= smem_limit) {
            // a block with very few warps cannot hide latency: prefer more tree threads
            if (rw * tt < 8 && tt < 16 && user.tree_threads <= 0 && rw_hi * tt >= 8) break;
            best = p;
            have = true;
            break;
          }
        }
      }
    }
  }
  if (!have) return "no launch shape fits the shared-memory budget for this forest";

  LaunchPlan &p = best;
  const int64_t rows_per_block = (int64_t)p.row_warps * 32 * p.rows_per_lane;
  p.grid_x = (n_rows + rows_per_block - 1) / rows_per_block;
  int64_t chunks = 1;
  if (user.tree_chunks > 0) {
    chunks = user.tree_chunks;
  } else if (p.grid_x < 2 * (int64_t)num_sms) {
    // A batch too small to fill the GPU with row tiles: split the forest into tree chunks
    // (grid.y) where that shortens the launch.  Cost model in microseconds, fitted to
    // measurements on B200 with a cold L2: a group costs about 2.5 (its bulk copy, one in
    // flight ahead of the walk) or, when a warp walks several columns of it, 0.75 per
    // column per full block of warps; a block pays about three to stage its rows; the
    // second pass (a launch and a small kernel) about six as soon as there is more than
    // one chunk.
    p.smem_bytes = (int32_t)smem_needed(fs, p);
    const int64_t threads = (int64_t)p.row_warps * p.tree_threads * 32;
    const int64_t resident = std::max<int64_t>(1, std::min<int64_t>((233472 - 1024) / (p.smem_bytes + 1024), 2048 / threads));
    const int64_t slots = resident * num_sms;
    const double group_cost = std::max(2.5, 0.75 * (16.0 / p.tree_threads) * (double)threads / 1024.0);
    double best_cost = -1.0;
    for (int64_t c = 1; c <= std::min<int64_t>(fs.num_groups, 64); ++c) {
      const int64_t per_block = (fs.num_groups + c - 1) / c;
      const int64_t waves = (p.grid_x * c + slots - 1) / slots;
      const double cost = (double)waves * ((double)per_block * group_cost + 3.0) + (c > 1 ? 6.0 : 0.0);
      if (best_cost < 0 || cost < best_cost - 1e-9) {
        best_cost = cost;
        chunks = c;
      }
    }
  }
  chunks = std::max<int64_t>(1, std::min<int64_t>(chunks, fs.num_groups));
  chunks = std::min<int64_t>(chunks, 65535);
  p.groups_per_chunk = (int32_t)((fs.num_groups + chunks - 1) / chunks);
  p.chunks = (int32_t)((fs.num_groups + p.groups_per_chunk - 1) / p.groups_per_chunk);
  p.threads = p.row_warps * p.tree_threads * 32;
  p.smem_bytes = (int32_t)smem_needed(fs, p);
  *out = p;
  return "";
}

} // namespace tb
