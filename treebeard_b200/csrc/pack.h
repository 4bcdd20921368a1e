// Forest -> packed node-tile buffers ("forest-to-buffer lowering").
//
// Covers the ground of the reference's serializers and tiling utilities
// (array layout: src/include/DecisionForest.h:292-315 and
// src/utils/TreeTilingUtils.cpp:1067-1112; sparse layout:
// src/include/DecisionForest.h:595-629 and src/utils/TreeTilingUtils.cpp:1256-1338;
// reorg layout: src/gpu/ReorgForestRepresentation.cpp:186-275; uniform tiling:
// src/mlir/UniformTilingTransformation.cpp:148-195; tile shapes and look-up table:
// src/utils/TreeTilingUtils.cpp:1749-2018; sorting trees by depth:
// src/mlir/GPUAutoSchedule.cpp:42-224) with a layout designed for the B200 kernels:
//
//  * Trees are sorted by (depth, size) and cut into GROUPS of 16.  Inside a group the
//    16 trees are interleaved slot-major: element (slot s, tree column c) sits at
//    index s*16 + c.  A warp whose lanes walk different columns therefore touches
//    16 distinct 8-byte bank pairs of shared memory per load, whatever slots the
//    lanes are at.
//  * Every group is a contiguous, 16-byte aligned byte range, so one bulk async copy
//    stages it into shared memory.
//  * sparse: 8-byte tile {fp32 threshold[ts], u16 feature[ts], ..., u16 child};
//    children of a tile are adjacent, next = child + k.
//  * array: implicit children, next = (ts+1)*n + 1 + k, trees padded to the complete
//    shape of the group's depth.
//  * reorg: as array with ts = 1, but thresholds and feature indices in separate
//    planes (6 bytes per node).
//  * Leaves never end a walk early: a leaf slot holds its value in the threshold
//    field, names the sentinel feature (index num_features, whose staged value is
//    -inf so "x < value" always holds) and leads back to itself (sparse) or down a
//    chain of copies (array/reorg).  Every tree of a group is walked for exactly the
//    group's depth; the slot reached holds the leaf value.
#pragma once
#include "forest.h"

#include <cstdint>
#include <string>
#include <vector>

namespace tb {

constexpr int kGroupTrees = 16;
constexpr int kMaxTileSize = 4;

enum Representation : int32_t { kSparse = 0, kArray = 1, kReorg = 2 };

struct GroupMeta {
  uint64_t byte_off; // offset of the group in the blob (multiple of 16)
  uint32_t slots;    // tile slots per tree column
  uint32_t depth;    // walk steps (tile levels) for this group
};

struct PackedForest {
  int32_t representation = kSparse;
  int32_t tile_size = 1;
  int32_t tile_bytes = 8;     // bytes of one tile (sparse/array); reorg: 6 per node
  int32_t num_features = 0, num_classes = 0, transform = 0;
  double initial_value = 0.0;
  int64_t num_trees = 0, num_nodes = 0;
  int32_t max_depth = 0;          // decision levels of the deepest tree
  uint64_t max_group_bytes = 0;
  std::vector<GroupMeta> groups;
  std::vector<uint8_t> blob;        // all groups back to back
  std::vector<int16_t> tree_class;  // [groups*16] class id of each column
  std::vector<int32_t> tree_index;  // [groups*16] original tree index, -1 = filler
  std::vector<uint64_t> orig_off;   // per group: offset into orig_node
  std::vector<int32_t> orig_node;   // per (slot, column[, exit]) original node id
  // tile-shape look-up table: lut[shape * (1 << tile_size) + outcome_bits] = child
  // number; bit i of outcome_bits is "x < threshold" of tile node i (LSB = node 0,
  // as the reference's GPU code packs them: src/mlir/CodeGenStateMachine.cpp:806-811)
  std::vector<int8_t> lut;
  int32_t num_shapes = 0;
};

struct PackOptions {
  int32_t representation = kSparse;
  int32_t tile_size = 1;
};

// Returns an empty string on success, else the reason.
std::string pack_forest(const Forest &f, const PackOptions &opt, PackedForest *out);

// Host-side interpreter of the packed buffers: the slot arithmetic the kernels use,
// executed on the CPU to verify the packer.  Writes the original node id of the leaf
// selected for every (row, tree).  It is a verification utility for the layout; no
// prediction path calls it.
void walk_packed_on_host(const PackedForest &p, const float *rows, int64_t n_rows, int64_t ld,
                         int32_t *leaf_ids, float *sums /* n_rows x max(1,C), may be null */);

} // namespace tb
