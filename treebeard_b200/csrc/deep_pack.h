// "One tree per stage": the packed layout for forests of DEEP trees (9 .. 12 decision
// levels), whose 16-tree groups are far too large for the shared-memory stages of the
// general kernel -- the reference then walks such trees from global memory
// (src/gpu/GPURepresentations.cpp:630-715 caches a tree only when it fits).
//
// Every tree becomes a complete tree of its pair's depth D (trees are sorted by depth and
// taken two at a time; a pair is what one thread walks in lock-step), stored as planes of
// 2^D elements per tree, 16 KB at D = 12:
//
//   node plane   u32 [2^D]  word i = node with 1-based heap index i (children 2i, 2i+1, an
//                           aligned 8-byte pair); (feature index << 16) | threshold key;
//                           word 0 is unused
//   leaf plane   f32 [2^D]  value of leaf j = i - 2^D after D steps
//   exact plane  f32 [2^D]  fp32 thresholds, indexed like the node plane (global memory only)
//
// Rows are staged as the 15-bit order-preserving keys of quant_pack.h, so a block holds
// 32 x row_warps rows (512 for 128 features) next to a ring of whole-tree pieces; key ties
// are resolved on the exact fp32 values, which keeps leaf selection that of the fp32 walk.
// A leaf above the bottom level is a chain of pass-through nodes (sentinel feature, key 0:
// always left) ending in the leaf slot that holds its value.
#pragma once
#include "forest.h"
#include "quant_pack.h"

#include <cstdint>
#include <string>
#include <vector>

namespace tb {

constexpr int kDeepMaxDepth = 12;
constexpr int kDeepMinDepth = 2; // pieces of at least 16 bytes

struct DeepForest {
  int32_t num_features = 0, transform = 0;
  double initial_value = 0.0;
  int64_t num_trees = 0, num_nodes = 0;
  int32_t max_depth = 0;
  std::vector<QuantGroup> pairs;    // elem_off of tree 0 of the pair (tree 1 follows at + slots)
  std::vector<uint32_t> node_plane; // key field is filled on the device at upload
  std::vector<float> leaf_plane;
  std::vector<float> exact_plane;
  std::vector<int32_t> orig_leaf;   // original node id per leaf-plane element
  std::vector<int32_t> tree_index;  // [pairs*2] original tree index, -1 = filler
  std::vector<float> lo, scale;     // per feature (+ sentinel entry)
};

// Empty string on success; fails for multiclass forests, trees deeper than kDeepMaxDepth
// or non-finite thresholds.
std::string pack_deep(const Forest &f, DeepForest *out);

// Host interpreter of the packed planes (layout verification only).
void walk_deep_on_host(const DeepForest &q, const float *rows, int64_t n_rows, int64_t ld,
                       int32_t *leaf_ids, float *sums, int64_t *ties);

} // namespace tb
