#include "quant_pack.h"

#include <algorithm>
#include <limits>
#include <numeric>

namespace tb {

std::string quant_feature_ranges(const Forest &f, float span, std::vector<float> *lo_out, std::vector<float> *scale_out,
                                 bool lattice) {
  const int F = f.num_features;
  std::vector<float> lo(F + 1, std::numeric_limits<float>::infinity());
  std::vector<float> hi(F + 1, -std::numeric_limits<float>::infinity());
  std::vector<char> whole(F + 1, 1); // every threshold of the feature is a whole number
  for (int64_t g = 0; g < f.num_nodes(); ++g) {
    if (!std::isfinite(f.thr[g])) return "non-finite threshold or leaf value";
    if (f.is_leaf(g)) continue;
    lo[f.feat[g]] = std::min(lo[f.feat[g]], f.thr[g]);
    hi[f.feat[g]] = std::max(hi[f.feat[g]], f.thr[g]);
    if (f.thr[g] != std::floor(f.thr[g]) || std::fabs(f.thr[g]) > 0x1p22f) whole[f.feat[g]] = 0;
  }
  lo_out->assign(F + 1, 0.f);
  scale_out->assign(F + 1, 0.f);
  for (int i = 0; i < F; ++i) {
    if (!(hi[i] >= lo[i])) continue; // feature not used by any split
    (*lo_out)[i] = lo[i];
    // a single threshold needs no range: any huge slope separates everything but x == t
    // the span is two steps short of the key range, which keeps the keys of the smallest and
    // the largest threshold off the two saturated keys under rounding
    float s = hi[i] > lo[i] ? span / (hi[i] - lo[i]) : 0x1p40f;
    if (!std::isfinite(s) || s <= 0.f) s = 0x1p40f;
    if (lattice && whole[i] && hi[i] - lo[i] <= span) {
      // whole-number thresholds: a whole-number slope puts each of them exactly on a key
      // (threshold - lo, the product and the sum are all exact in fp32)
      s = -(hi[i] > lo[i] ? std::floor(span / (hi[i] - lo[i])) : 1024.f);
    }
    (*scale_out)[i] = s;
  }
  return "";
}

std::string pack_quant(const Forest &f, QuantForest *out, bool lattice) {
  std::string err = validate(f);
  if (!err.empty()) return err;
  if (f.num_features > kQuantMaxFeatures) return "more than " + std::to_string(kQuantMaxFeatures) + " features";
  const int64_t T = f.num_trees();
  const int F = f.num_features;

  QuantForest &q = *out;
  q = QuantForest();
  q.num_features = F;
  q.transform = f.transform;
  q.num_classes = f.num_classes;
  q.initial_value = f.initial_value;
  q.num_trees = T;
  q.num_nodes = f.num_nodes();

  err = quant_feature_ranges(f, kKey15Span, &q.lo, &q.scale, lattice);
  if (!err.empty()) return err;

  std::vector<int32_t> depth(T);
  for (int64_t t = 0; t < T; ++t) {
    depth[t] = tree_depth(f, t);
    q.max_depth = std::max(q.max_depth, depth[t]);
  }
  if (q.max_depth > kQuantMaxDepth)
    return "trees deeper than " + std::to_string(kQuantMaxDepth) + " levels do not fit the key layout's stages";
  // columns in walking order: trees by depth -- within their class for a multiclass forest,
  // whose classes each fill whole groups -- and -1 for the filler columns
  std::vector<int64_t> order(T);
  std::iota(order.begin(), order.end(), 0);
  const bool multi = f.num_classes > 0;
  std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) {
    if (multi && f.class_id[a] != f.class_id[b]) return f.class_id[a] < f.class_id[b];
    return depth[a] < depth[b];
  });
  std::vector<int64_t> cols;
  if (multi) {
    size_t at = 0;
    for (int32_t cls = 0; cls < f.num_classes; ++cls) {
      const size_t begin = cols.size();
      while (at < order.size() && f.class_id[order[at]] == cls) cols.push_back(order[at++]);
      if (cols.size() == begin) cols.push_back(-1); // a class without trees still gets its group
      while (cols.size() % kQuantCols) cols.push_back(-1);
      q.group_class.insert(q.group_class.end(), (cols.size() - begin) / kQuantCols, cls);
    }
  } else {
    cols.assign(order.begin(), order.end());
    while (cols.size() % kQuantCols) cols.push_back(-1);
  }

  const int64_t G = (int64_t)cols.size() / kQuantCols;
  q.groups.resize(G);
  q.tree_index.assign(G * kQuantCols, -1);
  uint64_t elems = 0;
  for (int64_t g = 0; g < G; ++g) {
    uint32_t d = 1; // at least one level, so that every group has both halves of its planes
    for (int c = 0; c < kQuantCols; ++c)
      if (cols[g * kQuantCols + c] >= 0) d = std::max<uint32_t>(d, depth[cols[g * kQuantCols + c]]);
    q.groups[g] = QuantGroup{elems, d, 1u << d};
    elems += (uint64_t)(1u << d) * kQuantCols;
  }
  const uint32_t pass_through = quant_feature_code((uint32_t)F) << 16; // sentinel feature, key 0: always left
  q.node_plane.assign(elems, pass_through);
  q.leaf_plane.assign(elems, 0.f);
  q.exact_plane.assign(elems, 0.f);
  q.orig_leaf.assign(elems, -1);

  for (int64_t g = 0; g < G; ++g) {
    const QuantGroup &gm = q.groups[g];
    for (int c = 0; c < kQuantCols; ++c) {
      const int64_t k = g * kQuantCols + c;
      if (cols[k] < 0) continue;
      const int64_t t = cols[k], a = f.tree_off[t];
      q.tree_index[k] = (int32_t)t;
      struct Item { int32_t node; uint32_t slot, level; };
      std::vector<Item> stack{{0, 0, 0}};
      while (!stack.empty()) {
        const Item it = stack.back();
        stack.pop_back();
        if (f.left[a + it.node] < 0) {
          // leftmost descendant on the bottom level holds the value
          const uint64_t bottom = ((uint64_t)it.slot + 1) * (1ull << (gm.depth - it.level)) - 1;
          const uint64_t leaf = bottom - (gm.slots - 1);
          q.leaf_plane[quant_leaf_elem(gm, leaf, c)] = f.thr[a + it.node];
          q.orig_leaf[quant_leaf_elem(gm, leaf, c)] = it.node;
          continue;
        }
        const int32_t ft = f.feat[a + it.node];
        const float thr = f.thr[a + it.node];
        const uint64_t e = gm.elem_off + (uint64_t)quant_plane_slot(it.slot, it.level, gm.depth) * kQuantCols + c;
        q.node_plane[e] = (quant_feature_code((uint32_t)ft) << 16) | quant_threshold_key15(thr, q.lo[ft], q.scale[ft]);
        ++q.num_splits;
        if (thr == std::floor(thr) && !(q.scale[ft] < 0.f)) ++q.whole_number_splits;
        q.exact_plane[e] = thr;
        stack.push_back({f.left[a + it.node], 2 * it.slot + 1, it.level + 1});
        stack.push_back({f.right[a + it.node], 2 * it.slot + 2, it.level + 1});
      }
    }
  }
  return "";
}

void walk_quant_on_host(const QuantForest &q, const float *rows, int64_t n_rows, int64_t ld,
                        int32_t *leaf_ids, float *sums, int64_t *ties) {
  int64_t tie_count = 0;
  const int F = q.num_features;
  std::vector<uint16_t> keys(F + 1);
  for (int64_t r = 0; r < n_rows; ++r) {
    const float *row = rows + r * ld;
    for (int i = 0; i < F; ++i) keys[i] = quant_key15(row[i], q.lo[i], q.scale[i]);
    keys[F] = (uint16_t)kKey15Max;
    float acc = 0.f;
    const int C = q.num_classes;
    if (sums && C > 0) std::fill(sums + r * C, sums + (r + 1) * C, 0.f);
    for (size_t g = 0; g < q.groups.size(); ++g) {
      const QuantGroup &gm = q.groups[g];
      for (int c = 0; c < kQuantCols; ++c) {
        const int32_t t = q.tree_index[g * kQuantCols + c];
        if (t < 0) continue;
        uint32_t n = 0;
        for (uint32_t d = 0; d < gm.depth; ++d) {
          const uint64_t e = gm.elem_off + (uint64_t)quant_plane_slot(n, d, gm.depth) * kQuantCols + c;
          const uint32_t node = q.node_plane[e];
          const uint32_t ft = quant_feature_of_code(node >> 16), kt = node & 0x7fffu, kx = keys[ft];
          bool right = kx < kt;
          if (kx == kt) {
            ++tie_count;
            right = !(row[ft] < q.exact_plane[e]);
          }
          n = 2 * n + 1 + (right ? 1 : 0);
        }
        const uint64_t e = quant_leaf_elem(gm, n - (gm.slots - 1), c);
        acc += q.leaf_plane[e];
        if (sums && C > 0) sums[r * C + q.group_class[g]] += q.leaf_plane[e];
        if (leaf_ids) leaf_ids[r * q.num_trees + t] = q.orig_leaf[e];
      }
    }
    if (sums && C == 0) sums[r] = acc;
  }
  if (ties) *ties = tie_count;
}

} // namespace tb
