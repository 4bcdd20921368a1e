// XGBoost JSON model -> Forest.
//
// Follows the reference's front end (src/json/xgboostparser.h): base score and
// objective rules :94-114 (binary:logistic => initial value -ln(1/base_score - 1) and a
// sigmoid; reg:squarederror => identity; multi:softmax => class argmax), learner fields
// :116-145, class id per tree from tree_info :171, per-tree arrays :177-219
// (split_conditions narrowed to the fp32 threshold type, default_left ignored, root
// parent sentinel 2147483647).
#include "loaders.h"

#include "json.h"

#include <cmath>
#include <fstream>
#include <sstream>

namespace tb {

std::string load_xgboost_json(const std::string &path, Forest *out) {
  std::ifstream fin(path, std::ios::binary);
  if (!fin) return "cannot open " + path;
  std::stringstream ss;
  ss << fin.rdbuf();
  const std::string text = ss.str();
  try {
    const json::Value root = json::parse(text);
    const json::Value &learner = root.at("learner");
    const json::Value &params = learner.at("learner_model_param");
    const double base_score = params.at("base_score").number();
    const std::string objective = learner.at("objective").at("name").string();
    Forest f;
    if (objective == "binary:logistic") {
      f.initial_value = -std::log(1.0 / base_score - 1.0);
      f.transform = kSigmoid;
    } else if (objective == "reg:squarederror") {
      f.initial_value = base_score;
      f.transform = kIdentity;
    } else if (objective == "multi:softmax") {
      f.initial_value = base_score;
      f.transform = kSoftMax;
    } else {
      return "unknown objective \"" + objective + "\"";
    }
    f.num_classes = (int32_t)params.at("num_class").number();
    int32_t num_features = 0;
    if (params.has("num_feature")) num_features = (int32_t)params.at("num_feature").number();
    if (num_features <= 0 && learner.has("feature_types"))
      num_features = (int32_t)learner.at("feature_types").array().size();

    const json::Value &model = learner.at("gradient_booster").at("model");
    const json::Array &trees = model.at("trees").array();
    const json::Array &tree_info = model.at("tree_info").array();
    const size_t num_trees = (size_t)model.at("gbtree_model_param").at("num_trees").number();
    if (num_trees != trees.size() || num_trees != tree_info.size())
      return "num_trees does not match the trees / tree_info arrays";
    for (size_t t = 0; t < trees.size(); ++t) {
      const json::Value &tr = trees[t];
      const json::Array &lc = tr.at("left_children").array();
      const json::Array &rc = tr.at("right_children").array();
      const json::Array &sc = tr.at("split_conditions").array();
      const json::Array &si = tr.at("split_indices").array();
      const size_t n = (size_t)tr.at("tree_param").at("num_nodes").number();
      if (lc.size() != n || rc.size() != n || sc.size() != n || si.size() != n)
        return "tree " + std::to_string(t) + ": node arrays do not match num_nodes";
      if (tr.at("tree_param").has("num_feature"))
        num_features = std::max(num_features, (int32_t)tr.at("tree_param").at("num_feature").number());
      for (size_t i = 0; i < n; ++i) {
        f.left.push_back((int32_t)lc[i].number());
        f.right.push_back((int32_t)rc[i].number());
        f.feat.push_back((int32_t)si[i].number());
        f.thr.push_back((float)sc[i].number());
      }
      f.tree_off.push_back((int64_t)f.left.size());
      f.class_id.push_back((int32_t)tree_info[t].number());
    }
    f.num_features = num_features;
    if (f.num_classes == 0) std::fill(f.class_id.begin(), f.class_id.end(), 0);
    *out = std::move(f);
  } catch (const std::exception &e) {
    return path + ": " + e.what();
  }
  return "";
}

} // namespace tb
