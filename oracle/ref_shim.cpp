// TEST INFRASTRUCTURE -- thin C shim over the reference's own, unmodified
// ground-truth walker.  The reference header src/include/DecisionForest.h is
// included from the reference checkout at build time (it is never copied into
// this repository); the resulting library lands in oracle/_ref/ and is used to
// validate the C restatement in walk.c and, optionally, as the timed CPU
// baseline ("kind": "reference").
//
// The forest is rebuilt through the header's public construction API exactly as
// the reference's XGBoost front end does it (src/json/xgboostparser.h:177-219:
// NewNode(threshold, featureIndex) per node, then left/right/parent links, root
// parent -1; class id per tree; initial value, transformation and class count on
// the forest), and predictions come from DecisionForest::Predict_Float
// (src/include/DecisionForest.h:504-536).
#include "DecisionForest.h"

#include <cstdint>
#include <vector>

using mlir::decisionforest::DecisionForest;
using mlir::decisionforest::PredictionTransformation;

extern "C" {

void *tbref_forest_create(int64_t num_trees, const int64_t *tree_off,
                          const int32_t *left, const int32_t *right,
                          const int32_t *feat, const float *thr,
                          const int32_t *class_id, int32_t num_classes,
                          int32_t transform, double initial_value,
                          int32_t num_features) {
  auto *forest = new DecisionForest(initial_value);
  for (int32_t i = 0; i < num_features; ++i)
    forest->AddFeature(std::to_string(i), "float");
  forest->SetNumClasses(num_classes);
  forest->SetPredictionTransformation(
      transform == 0   ? PredictionTransformation::kIdentity
      : transform == 1 ? PredictionTransformation::kSigmoid
                       : PredictionTransformation::kSoftMax);
  for (int64_t t = 0; t < num_trees; ++t) {
    auto &tree = forest->NewTree();
    tree.SetNumberOfFeatures(num_features);
    tree.SetTreeScalingFactor(1.0);
    const int64_t base = tree_off[t], n = tree_off[t + 1] - base;
    std::vector<int64_t> parent(n, -1);
    for (int64_t i = 0; i < n; ++i)
      tree.NewNode((double)thr[base + i], feat[base + i]);
    for (int64_t i = 0; i < n; ++i) {
      if (left[base + i] != -1) {
        tree.SetNodeLeftChild(i, left[base + i]);
        parent[left[base + i]] = i;
      }
      if (right[base + i] != -1) {
        tree.SetNodeRightChild(i, right[base + i]);
        parent[right[base + i]] = i;
      }
    }
    for (int64_t i = 0; i < n; ++i)
      tree.SetNodeParent(i, parent[i]);
    tree.SetClassId(class_id ? class_id[t] : 0);
  }
  return forest;
}

void tbref_forest_free(void *f) { delete static_cast<DecisionForest *>(f); }

int tbref_predict(void *f, const float *rows, int64_t n_rows, int64_t ld,
                  int32_t num_features, float *out) {
  auto *forest = static_cast<DecisionForest *>(f);
#pragma omp parallel
  {
    std::vector<float> row(num_features);
#pragma omp for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
      row.assign(rows + r * ld, rows + r * ld + num_features);
      out[r] = forest->Predict_Float(row);
    }
  }
  return 0;
}

// Per-tree selected leaf value, for cross-checking the restatement's walk.
int tbref_tree_outputs(void *f, const float *rows, int64_t n_rows, int64_t ld,
                       int32_t num_features, float *out /* n_rows x T */) {
  auto *forest = static_cast<DecisionForest *>(f);
  const int64_t T = (int64_t)forest->NumTrees();
  std::vector<float> row(num_features);
  for (int64_t r = 0; r < n_rows; ++r) {
    row.assign(rows + r * ld, rows + r * ld + num_features);
    for (int64_t t = 0; t < T; ++t)
      out[r * T + t] = forest->GetTree(t).PredictTree_Float(row);
  }
  return 0;
}
}
