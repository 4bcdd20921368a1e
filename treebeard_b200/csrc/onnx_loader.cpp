// ONNX TreeEnsembleRegressor / TreeEnsembleClassifier -> Forest.
//
// Covers what the reference's ONNX front end accepts (src/json/onnxmodelparser.h:52-177:
// a graph with a single tree-ensemble node, one base value, post_transform NONE /
// LOGISTIC / SOFTMAX, one comparison mode per model out of BRANCH_LT / BRANCH_LEQ /
// BRANCH_GT / BRANCH_GEQ, no missing-value tracks; :220-374: true branch = left child,
// leaf values from the target/class weight tables, one class per tree).
//
// The file is read with a small protobuf wire-format reader that follows the message
// layout of onnx.proto (ModelProto.graph = 7, GraphProto.node = 1, NodeProto.op_type = 4
// and .attribute = 5, AttributeProto name = 1, f = 2, i = 3, s = 4, floats = 7, ints = 8,
// strings = 9); no protobuf library is needed.
//
// Every comparison mode is rewritten, exactly, into the kernels' single predicate
// "x < t goes left":  x <= t  <=>  x < nextafter(t, +inf);  x >= t and x > t are the
// negations of x < t and x <= t, i.e. the same test with the children swapped.
#include "loaders.h"

#include <algorithm>
#include <cmath>
#include <cstring>
#include <fstream>
#include <limits>
#include <map>
#include <set>
#include <sstream>

namespace tb {
namespace {

struct Wire {
  const uint8_t *p, *end;
  bool ok = true;
  uint64_t varint() {
    uint64_t v = 0;
    int shift = 0;
    while (p < end && shift < 64) {
      const uint8_t c = *p++;
      v |= (uint64_t)(c & 0x7f) << shift;
      if (c < 0x80) return v;
      shift += 7;
    }
    ok = false;
    return 0;
  }
  // next field: number, wire type, and either a scalar or a byte range
  bool next(uint32_t *field, uint32_t *type, uint64_t *scalar, const uint8_t **b, const uint8_t **e) {
    if (p >= end || !ok) return false;
    const uint64_t key = varint();
    *field = (uint32_t)(key >> 3);
    *type = (uint32_t)(key & 7);
    switch (*type) {
    case 0: *scalar = varint(); break;
    case 1: if (end - p < 8) { ok = false; return false; } std::memcpy(scalar, p, 8); p += 8; break;
    case 5: { if (end - p < 4) { ok = false; return false; } uint32_t v; std::memcpy(&v, p, 4); *scalar = v; p += 4; break; }
    case 2: {
      const uint64_t len = varint();
      if (!ok || (uint64_t)(end - p) < len) { ok = false; return false; }
      *b = p;
      *e = p + len;
      p += len;
      break;
    }
    default: ok = false; return false;
    }
    return ok;
  }
};

struct Attribute {
  std::string name, s;
  float f = 0.f;
  int64_t i = 0;
  std::vector<float> floats;
  std::vector<int64_t> ints;
  std::vector<std::string> strings;
};

bool parse_attribute(const uint8_t *b, const uint8_t *e, Attribute *a) {
  Wire w{b, e};
  uint32_t field, type;
  uint64_t v;
  const uint8_t *sb = nullptr, *se = nullptr;
  while (w.next(&field, &type, &v, &sb, &se)) {
    switch (field) {
    case 1: if (type == 2) a->name.assign(sb, se); break;
    case 2: if (type == 5) { uint32_t u = (uint32_t)v; std::memcpy(&a->f, &u, 4); } break;
    case 3: if (type == 0) a->i = (int64_t)v; break;
    case 4: if (type == 2) a->s.assign(sb, se); break;
    case 7:
      if (type == 5) { uint32_t u = (uint32_t)v; float x; std::memcpy(&x, &u, 4); a->floats.push_back(x); }
      else if (type == 2) for (const uint8_t *q = sb; q + 4 <= se; q += 4) { float x; std::memcpy(&x, q, 4); a->floats.push_back(x); }
      break;
    case 8:
      if (type == 0) a->ints.push_back((int64_t)v);
      else if (type == 2) { Wire pw{sb, se}; while (pw.p < pw.end && pw.ok) a->ints.push_back((int64_t)pw.varint()); }
      break;
    case 9: if (type == 2) a->strings.emplace_back(sb, se); break;
    default: break;
    }
  }
  return w.ok;
}

} // namespace

std::string load_onnx_file(const std::string &path, Forest *out) { return load_onnx_file(path, 0, out); }

std::string load_onnx_file(const std::string &path, int32_t num_features_hint, Forest *out) {
  std::ifstream fin(path, std::ios::binary);
  if (!fin) return "cannot open " + path;
  std::stringstream ss;
  ss << fin.rdbuf();
  const std::string data = ss.str();
  const uint8_t *base = reinterpret_cast<const uint8_t *>(data.data());

  // ModelProto -> graph -> nodes
  Wire model{base, base + data.size()};
  uint32_t field, type;
  uint64_t v;
  const uint8_t *b = nullptr, *e = nullptr;
  const uint8_t *gb = nullptr, *ge = nullptr;
  while (model.next(&field, &type, &v, &b, &e))
    if (field == 7 && type == 2) { gb = b; ge = e; }
  if (!model.ok || !gb) return path + ": not an ONNX model (no graph)";
  std::vector<std::pair<const uint8_t *, const uint8_t *>> nodes;
  Wire graph{gb, ge};
  while (graph.next(&field, &type, &v, &b, &e))
    if (field == 1 && type == 2) nodes.push_back({b, e});
  if (!graph.ok) return path + ": malformed graph";
  if (nodes.size() != 1) return path + ": only graphs with a single node are supported";

  std::string op_type;
  std::map<std::string, Attribute> attrs;
  Wire node{nodes[0].first, nodes[0].second};
  while (node.next(&field, &type, &v, &b, &e)) {
    if (field == 4 && type == 2) op_type.assign(b, e);
    if (field == 5 && type == 2) {
      Attribute a;
      if (!parse_attribute(b, e, &a)) return path + ": malformed attribute";
      attrs[a.name] = std::move(a);
    }
  }
  if (!node.ok) return path + ": malformed node";
  const bool classifier = op_type == "TreeEnsembleClassifier";
  if (!classifier && op_type != "TreeEnsembleRegressor")
    return path + ": operator \"" + op_type + "\" is not a tree ensemble";

  auto ints = [&](const char *n) -> const std::vector<int64_t> & { return attrs[n].ints; };
  const auto &tree_ids = ints("nodes_treeids"), &node_ids = ints("nodes_nodeids"), &feat_ids = ints("nodes_featureids");
  const auto &true_ids = ints("nodes_truenodeids"), &false_ids = ints("nodes_falsenodeids");
  const auto &values = attrs["nodes_values"].floats;
  const auto &modes = attrs["nodes_modes"].strings;
  const size_t n = node_ids.size();
  if (n == 0 || tree_ids.size() != n || feat_ids.size() != n || true_ids.size() != n || false_ids.size() != n ||
      values.size() != n || modes.size() != n)
    return path + ": node attribute arrays are missing or of different lengths";
  for (int64_t t : ints("nodes_missing_value_tracks_true"))
    if (t != 0) return path + ": missing-value tracks are not supported";
  if (attrs.count("aggregate_function") && !attrs["aggregate_function"].s.empty() && attrs["aggregate_function"].s != "SUM")
    return path + ": only the SUM aggregate function is supported";

  // one comparison mode for the whole model
  std::set<std::string> cmp;
  for (const std::string &m : modes)
    if (m != "LEAF") cmp.insert(m);
  if (cmp.size() > 1) return path + ": mixed comparison modes are not supported";
  const std::string mode = cmp.empty() ? "BRANCH_LT" : *cmp.begin();
  bool swap_children, bump_threshold;
  if (mode == "BRANCH_LT") { swap_children = false; bump_threshold = false; }
  else if (mode == "BRANCH_LEQ") { swap_children = false; bump_threshold = true; }
  else if (mode == "BRANCH_GEQ" || mode == "BRANCH_GTE") { swap_children = true; bump_threshold = false; }
  else if (mode == "BRANCH_GT") { swap_children = true; bump_threshold = true; }
  else return path + ": comparison mode " + mode + " is not supported";

  Forest f;
  const std::string post = attrs.count("post_transform") ? attrs["post_transform"].s : "NONE";
  if (post == "NONE" || post.empty()) f.transform = kIdentity;
  else if (post == "LOGISTIC") f.transform = kSigmoid;
  else if (post == "SOFTMAX") f.transform = kSoftMax;
  else return path + ": post_transform " + post + " is not supported";
  const auto &base_values = attrs["base_values"].floats;
  f.initial_value = 0.0;
  if (!base_values.empty()) {
    for (float bv : base_values)
      if (bv != base_values[0]) return path + ": differing base values per output are not supported";
    f.initial_value = base_values[0];
  }

  // leaf weights: regressor target_* tables, classifier class_* tables
  const char *pre = classifier && attrs.count("class_weights") ? "class_" : "target_";
  const auto &w_tree = ints((std::string(pre) + "treeids").c_str());
  const auto &w_node = ints((std::string(pre) + "nodeids").c_str());
  const auto &w_ids = ints((std::string(pre) + "ids").c_str());
  const auto &w_val = attrs[std::string(pre) + "weights"].floats;
  if (w_tree.size() != w_val.size() || w_node.size() != w_val.size() || w_ids.size() != w_val.size())
    return path + ": leaf weight tables are of different lengths";

  // trees in order of first appearance; nodes addressed by (tree id, node id)
  std::map<int64_t, int64_t> tree_slot;
  std::vector<int64_t> tree_order;
  std::vector<std::map<int64_t, size_t>> node_row; // per tree: node id -> row in the attribute arrays
  for (size_t i = 0; i < n; ++i) {
    auto it = tree_slot.find(tree_ids[i]);
    if (it == tree_slot.end()) {
      it = tree_slot.emplace(tree_ids[i], (int64_t)tree_order.size()).first;
      tree_order.push_back(tree_ids[i]);
      node_row.emplace_back();
    }
    node_row[it->second][node_ids[i]] = i;
  }
  const size_t T = tree_order.size();
  std::vector<std::map<int64_t, float>> leaf_value(T);
  std::vector<std::set<int64_t>> tree_classes(T);
  for (size_t i = 0; i < w_val.size(); ++i) {
    auto it = tree_slot.find(w_tree[i]);
    if (it == tree_slot.end()) return path + ": weight for an unknown tree";
    leaf_value[it->second][w_node[i]] += w_val[i];
    tree_classes[it->second].insert(w_ids[i]);
  }

  int64_t max_feature = -1, max_class = -1;
  for (size_t t = 0; t < T; ++t) {
    const auto &rows = node_row[t];
    auto root = rows.find(0);
    if (root == rows.end()) return path + ": tree without node 0";
    // depth-first numbering from the root, parent before children
    std::vector<std::pair<int64_t, int32_t>> stack{{0, -1}}; // (onnx node id, index of parent slot to patch)
    const int64_t first = (int64_t)f.left.size();
    std::vector<int> patch_right; // per emitted node: 1 if the pending link is the right child
    struct Pending { int64_t id; int32_t parent; bool right; };
    std::vector<Pending> work{{0, -1, false}};
    while (!work.empty()) {
      const Pending cur = work.back();
      work.pop_back();
      auto it = rows.find(cur.id);
      if (it == rows.end()) return path + ": child node id not found";
      const size_t i = it->second;
      const int32_t idx = (int32_t)((int64_t)f.left.size() - first);
      if (idx > (1 << 24)) return path + ": tree too large (cycle?)";
      if (cur.parent >= 0) (cur.right ? f.right : f.left)[first + cur.parent] = idx;
      f.left.push_back(-1);
      f.right.push_back(-1);
      if (modes[i] == "LEAF") {
        f.feat.push_back(0);
        auto lv = leaf_value[t].find(cur.id);
        f.thr.push_back(lv == leaf_value[t].end() ? 0.f : lv->second);
      } else {
        float thr = values[i];
        if (bump_threshold) thr = std::nextafterf(thr, std::numeric_limits<float>::infinity());
        f.feat.push_back((int32_t)feat_ids[i]);
        f.thr.push_back(thr);
        max_feature = std::max(max_feature, feat_ids[i]);
        const int64_t t_id = true_ids[i], f_id = false_ids[i];
        // true branch = left child (reference: onnxmodelparser.h:226-227); swapped for >= / >
        work.push_back({swap_children ? t_id : f_id, idx, true});
        work.push_back({swap_children ? f_id : t_id, idx, false});
      }
    }
    f.tree_off.push_back((int64_t)f.left.size());
    if (classifier) {
      if (tree_classes[t].size() > 1) return path + ": a tree that votes for several classes is not supported";
      const int64_t c = tree_classes[t].empty() ? 0 : *tree_classes[t].begin();
      f.class_id.push_back((int32_t)c);
      max_class = std::max(max_class, c);
    } else {
      if (tree_classes[t].size() > 1 || (!tree_classes[t].empty() && *tree_classes[t].begin() != 0))
        return path + ": multi-target regressors are not supported";
      f.class_id.push_back(0);
    }
  }
  f.num_features = (int32_t)std::max<int64_t>(num_features_hint, max_feature + 1);
  if (classifier) {
    const size_t labels = attrs["classlabels_int64s"].ints.size() + attrs["classlabels_strings"].strings.size();
    const int64_t classes = std::max<int64_t>((int64_t)labels, max_class + 1);
    // a binary classifier whose trees all score one class is a single sigmoid output
    if (classes <= 2 && max_class <= 1 && f.transform != kSoftMax) {
      std::set<int32_t> used(f.class_id.begin(), f.class_id.end());
      if (used.size() == 1) {
        f.num_classes = 0;
        std::fill(f.class_id.begin(), f.class_id.end(), 0);
      } else {
        f.num_classes = (int32_t)classes;
      }
    } else {
      f.num_classes = (int32_t)classes;
      f.transform = kSoftMax;
    }
  }
  *out = std::move(f);
  return "";
}

} // namespace tb
