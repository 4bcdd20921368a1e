// "Reorg with 16-bit feature keys": the packed layout for forests over WIDE rows.
//
// When a row is so wide that a 32-row fp32 tile does not fit in shared memory (the
// reference simply stops caching rows beyond 1500 features,
// src/mlir/GPUAutoSchedule.cpp:803-806, and walks from global memory), rows are staged
// as 16-bit ORDER-PRESERVING KEYS instead, which halves the tile, and nodes shrink to
// 4 bytes.  The layout is the reorg idea (src/gpu/ReorgForestRepresentation.cpp:186-275:
// node-major planes, every tree padded to a complete tree, implicit children 2n+1+k)
// per group of 32 trees:
//
//   node plane   u32 [2^D slots][32 columns]   (feature code << 16) | threshold key
//   leaf plane   f32 [32 columns][2^D leaves]  leaf values, column-major: the leaves that a
//                                              warp needs for ONE tree lie within 1 KB
//   exact plane  f32 [2^D slots][32 columns]   fp32 thresholds (global memory only)
//
// Keys are 15-bit integers in [1024, 31743], i.e. bit patterns of positive, finite, normal
// half-precision numbers, so that the kernel can compare the low halves of two registers
// with ONE half2 comparison (no mask, no shift) and bit 15 of a node word is always 0.
// For feature f with thresholds in [lo_f, hi_f]:
//     key(v) = floor( min( max( fma(v - lo_f, -a_f, 31741), 1024 ), 31743 ) ),
//     a_f = 30715 / (hi_f - lo_f)
// a non-increasing map (NaN -> 1024, +inf -> 1024, -inf -> 31743; thresholds land in
// [1025, 31742]).  For a row value x and a threshold t of the same feature:
// key(x) > key(t)  =>  x < t  (left);  key(x) < key(t)  =>  x > t  (right);  equal keys
// decide nothing, and the kernel then compares the exact fp32 values.  Leaf selection is
// therefore exactly that of the fp32 walk; only speed depends on how often keys tie.
//
// The feature code of feature f is (f >> 1) * 64 + (f & 1): twice that is the byte offset of
// the feature's key inside a lane's column of the kernel's key tile, which keeps features
// 2m and 2m+1 of one row in one 32-bit word (see walk_quant.cuh).
//
// A leaf above the bottom level becomes a chain of pass-through nodes that name the
// sentinel feature (index num_features, staged key 31743) with key 0: always left.
#pragma once
#include "forest.h"

#include <cmath>
#include <cstdint>
#include <string>
#include <vector>

namespace tb {

constexpr int kQuantCols = 32;
constexpr int kQuantMaxDepth = 8; // node planes of at most 2^8 * 128 B = 32 KB: two 16 KB stages
constexpr int kQuantMaxFeatures = 2046; // feature codes (sentinel included) fit 16 bits

struct QuantGroup {
  uint64_t elem_off; // offset of the group's planes, in elements (same for all planes)
  uint32_t depth;    // decision levels; planes have 2^depth slots
  uint32_t slots;    // 2^depth
};

struct QuantForest {
  int32_t num_features = 0, transform = 0, num_classes = 0;
  double initial_value = 0.0;
  int64_t num_trees = 0, num_nodes = 0;
  int32_t max_depth = 0;
  std::vector<QuantGroup> groups;
  std::vector<uint32_t> node_plane; // key field is filled on the device at upload
  std::vector<float> leaf_plane;
  std::vector<float> exact_plane;
  std::vector<int32_t> orig_leaf;   // original node id per leaf-plane element
  std::vector<int32_t> tree_index;  // [groups*32] original tree index, -1 = filler
  std::vector<int32_t> group_class; // multiclass: the class every tree of the group votes for
  // split nodes in all, and those with a whole-number threshold on a feature that is not a
  // lattice feature (rows of integer-valued features tie with such thresholds all the time)
  int64_t num_splits = 0, whole_number_splits = 0;
  std::vector<float> lo, scale;     // per feature (+ sentinel entry)
};

// Slot of a split node in the node / exact planes.  Nodes are in level order (root 0,
// children 2n+1, 2n+2) except that the bottom decision level is pushed back by one slot:
// the first half of a plane (2^(depth-1) slots) then holds levels 0..depth-2 plus one unused
// slot, the second half exactly the bottom level, and each half is one contiguous piece
// for the kernel's staging ring.
inline uint32_t quant_plane_slot(uint32_t heap_slot, uint32_t level, uint32_t depth) {
  return level + 1 == depth ? heap_slot + 1 : heap_slot;
}

// Element of the leaf plane (and of orig_leaf) that holds leaf `leaf` of tree column `col`.
inline uint64_t quant_leaf_elem(const QuantGroup &g, uint64_t leaf, uint32_t col) {
  return g.elem_off + (uint64_t)col * g.slots + leaf;
}

// 15-bit keys of this layout and of the deep-tree layout (see the head of the file); same
// arithmetic on the device.
constexpr float kKey15Top = 31741.0f, kKey15Min = 1024.0f, kKey15Max = 31743.0f;
constexpr float kKey15Span = 30715.0f; // keys between the smallest and the largest threshold
// A NEGATIVE scale marks a lattice feature (see quant_feature_ranges): every threshold is a
// whole number and the slope |scale| is one too, so thresholds and whole-number row values
// land EXACTLY on keys (value - lo, the product and the sum are exact in fp32).  A whole-number
// row value x then has key(x) <= key(t) exactly when x >= t; any other row value gets
// floor + 1, which either decides like its neighbours or equals the node key (below).
inline uint16_t quant_key15(float v, float lo, float scale) {
  if (scale < 0.f) {
    float y = std::fmaf(v - lo, scale, kKey15Top);
    y = std::fmin(std::fmax(y, kKey15Min), kKey15Max);
    return v == std::floor(v) ? (uint16_t)y : (uint16_t)std::fmin(std::floor(y) + 1.0f, kKey15Max);
  }
  float y = std::fmaf(v - lo, -scale, kKey15Top);
  y = std::fmin(std::fmax(y, kKey15Min), kKey15Max); // fmax first: NaN becomes the smallest key
  return (uint16_t)std::floor(y);
}
// Key stored in a split node.  Ordinary features: the key of the threshold itself (equal keys
// decide nothing and go through the exact comparison).  Lattice features: one above it --
// whole-number rows at or above the threshold have keys up to the threshold's and go right by
// "row key < node key", whole-number rows below it have larger keys and go left, and only a
// row value that is not a whole number can meet the node key exactly (it lies within
// 1/|scale| of the threshold): the exact comparison then decides, as for any key tie.
inline uint16_t quant_threshold_key15(float t, float lo, float scale) {
  return scale < 0.f ? (uint16_t)(quant_key15(t, lo, scale) + 1) : quant_key15(t, lo, scale);
}
inline uint32_t quant_feature_code(uint32_t f) { return (f >> 1) * 64u + (f & 1u); }
inline uint32_t quant_feature_of_code(uint32_t code) { return (code >> 6) * 2u + (code & 1u); }

// Per-feature key parameters (entries 0..num_features; the last belongs to the sentinel
// feature): lo = smallest threshold of the feature, scale = span / (hi - lo), span being
// the number of key steps between the smallest and the largest threshold (kKey15Span here
// and in the deep-tree layout).  Fails on a non-finite threshold or leaf value.
// lattice: features whose thresholds are all whole numbers no more than `span` apart get a
// whole-number slope, stored NEGATED (see quant_key15): rows of integer-valued features, which
// equal thresholds all the time, then never need the exact comparison.
std::string quant_feature_ranges(const Forest &f, float span, std::vector<float> *lo, std::vector<float> *scale,
                                 bool lattice = false);

// lattice: allow lattice features (the kernel for narrow rows handles them).
// Empty string on success.  Fails (so that the caller can fall back to another layout)
// for trees deeper than kQuantMaxDepth or non-finite thresholds.  Multiclass forests are
// laid out class by class: every class is padded to whole groups (filler columns hold one
// pass-through tree with value 0), classes in increasing order, every class present, so a
// group belongs to one class (group_class).
std::string pack_quant(const Forest &f, QuantForest *out, bool lattice = false);

// Host interpreter of the packed planes (layout verification only).  sums: one value per
// row, or num_classes values per row for a multiclass forest.
void walk_quant_on_host(const QuantForest &q, const float *rows, int64_t n_rows, int64_t ld,
                        int32_t *leaf_ids, float *sums, int64_t *ties);

} // namespace tb
