// Host-side forest model.
//
// Plays the role of the reference's DecisionForest / DecisionTree::Node
// (src/include/DecisionForest.h:35-54, 179-264) as structure-of-arrays: leaf values
// live in `thr`, a node is a leaf when both children are -1.
#pragma once
#include <cstdint>
#include <string>
#include <vector>

namespace tb {

enum Transform : int32_t { kIdentity = 0, kSigmoid = 1, kSoftMax = 2 };

struct Forest {
  std::vector<int64_t> tree_off{0};
  std::vector<int32_t> left, right, feat;
  std::vector<float> thr;
  std::vector<int32_t> class_id;
  int32_t num_classes = 0;
  int32_t transform = kIdentity;
  double initial_value = 0.0;
  int32_t num_features = 0;

  int64_t num_trees() const { return (int64_t)tree_off.size() - 1; }
  int64_t num_nodes() const { return tree_off.back(); }
  bool is_leaf(int64_t g) const { return left[g] < 0 && right[g] < 0; }
};

// Checks indices, child links (every non-root node has exactly one parent, no
// cycles), feature range and class ids.  Returns an empty string when valid.
std::string validate(const Forest &f);

// Decision levels on the longest root-to-leaf path of tree t (a single leaf: 0).
int32_t tree_depth(const Forest &f, int64_t t);

// Threads for the packers' parallel loops: the machine's hardware threads (at most 32), not
// the OpenMP default, which process launchers commonly pin to 1 (torch.distributed.run
// exports OMP_NUM_THREADS=1 for its workers) although packing a large forest is the one
// host-side step that takes seconds.  TBK_PACK_THREADS overrides.
int pack_threads();

} // namespace tb
