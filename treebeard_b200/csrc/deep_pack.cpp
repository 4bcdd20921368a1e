#include "deep_pack.h"

#include <algorithm>
#include <numeric>

namespace tb {

std::string pack_deep(const Forest &f, DeepForest *out) {
  std::string err = validate(f);
  if (!err.empty()) return err;
  if (f.num_classes > 0) return "the deep-tree layout is implemented for single-output forests only";
  if (f.num_features > 65534) return "more than 65534 features";
  const int64_t T = f.num_trees();
  const int F = f.num_features;

  DeepForest &q = *out;
  q = DeepForest();
  q.num_features = F;
  q.transform = f.transform;
  q.initial_value = f.initial_value;
  q.num_trees = T;
  q.num_nodes = f.num_nodes();
  err = quant_feature_ranges(f, kKey15Span, &q.lo, &q.scale, /*lattice=*/true);
  if (!err.empty()) return err;

  std::vector<int32_t> depth(T);
#pragma omp parallel for schedule(dynamic, 64) num_threads(pack_threads())
  for (int64_t t = 0; t < T; ++t) depth[t] = tree_depth(f, t);
  for (int64_t t = 0; t < T; ++t) q.max_depth = std::max(q.max_depth, depth[t]);
  if (q.max_depth > kDeepMaxDepth)
    return "trees deeper than " + std::to_string(kDeepMaxDepth) + " levels do not fit a whole-tree stage";
  std::vector<int64_t> order(T);
  std::iota(order.begin(), order.end(), 0);
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return depth[a] < depth[b]; });

  const int64_t P = (T + 1) / 2;
  q.pairs.resize(P);
  q.tree_index.assign(P * 2, -1);
  uint64_t elems = 0;
  for (int64_t g = 0; g < P; ++g) {
    uint32_t d = kDeepMinDepth;
    for (int c = 0; c < 2 && 2 * g + c < T; ++c) d = std::max<uint32_t>(d, depth[order[2 * g + c]]);
    q.pairs[g] = QuantGroup{elems, d, 1u << d};
    elems += 2ull << d;
  }
  const uint32_t pass_through = (uint32_t)F << 16; // sentinel feature, key 0: always left
  q.node_plane.assign(elems, pass_through);
  q.leaf_plane.assign(elems, 0.f);
  q.exact_plane.assign(elems, 0.f);
  q.orig_leaf.assign(elems, -1);

#pragma omp parallel for schedule(dynamic, 16) num_threads(pack_threads())
  for (int64_t g = 0; g < P; ++g) {
    const QuantGroup &gm = q.pairs[g];
    for (int c = 0; c < 2; ++c) {
      const int64_t k = 2 * g + c;
      if (k >= T) break;
      const int64_t t = order[k], a = f.tree_off[t];
      const uint64_t base = gm.elem_off + (uint64_t)c * gm.slots;
      q.tree_index[k] = (int32_t)t;
      struct Item { int32_t node; uint32_t heap, level; };
      std::vector<Item> stack{{0, 1, 0}};
      while (!stack.empty()) {
        const Item it = stack.back();
        stack.pop_back();
        if (f.left[a + it.node] < 0) {
          // the leftmost descendant on the leaf level holds the value
          const uint64_t leaf = ((uint64_t)it.heap << (gm.depth - it.level)) - gm.slots;
          q.leaf_plane[base + leaf] = f.thr[a + it.node];
          q.orig_leaf[base + leaf] = it.node;
          continue;
        }
        const int32_t ft = f.feat[a + it.node];
        const float thr = f.thr[a + it.node];
            q.node_plane[base + it.heap] = ((uint32_t)ft << 16) | quant_threshold_key15(thr, q.lo[ft], q.scale[ft]);
        q.exact_plane[base + it.heap] = thr;
        stack.push_back({f.left[a + it.node], 2 * it.heap, it.level + 1});
        stack.push_back({f.right[a + it.node], 2 * it.heap + 1, it.level + 1});
      }
    }
  }
  return "";
}

void walk_deep_on_host(const DeepForest &q, const float *rows, int64_t n_rows, int64_t ld,
                       int32_t *leaf_ids, float *sums, int64_t *ties) {
  int64_t tie_count = 0;
  const int F = q.num_features;
  std::vector<uint16_t> keys(F + 1);
  for (int64_t r = 0; r < n_rows; ++r) {
    const float *row = rows + r * ld;
    for (int i = 0; i < F; ++i) keys[i] = quant_key15(row[i], q.lo[i], q.scale[i]);
    keys[F] = (uint16_t)kKey15Max;
    float acc = 0.f;
    for (size_t g = 0; g < q.pairs.size(); ++g) {
      const QuantGroup &gm = q.pairs[g];
      for (int c = 0; c < 2; ++c) {
        const int32_t t = q.tree_index[g * 2 + c];
        if (t < 0) continue;
        const uint64_t base = gm.elem_off + (uint64_t)c * gm.slots;
        uint32_t i = 1;
        for (uint32_t d = 0; d < gm.depth; ++d) {
          const uint32_t node = q.node_plane[base + i];
          const uint32_t ft = node >> 16, kt = node & 0xffffu, kx = keys[ft];
          bool right = kx < kt;
          if (kx == kt) {
            ++tie_count;
            right = !(row[ft] < q.exact_plane[base + i]);
          }
          i = 2 * i + (right ? 1 : 0);
        }
        const uint64_t e = base + (i - gm.slots);
        acc += q.leaf_plane[e];
        if (leaf_ids) leaf_ids[r * q.num_trees + t] = q.orig_leaf[e];
      }
    }
    if (sums) sums[r] = acc;
  }
  if (ties) *ties = tie_count;
}

} // namespace tb
