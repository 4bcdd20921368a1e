// Model file front ends.  Names follow the reference's forest-creator factory
// ("xgboost_json", "onnx_file": src/json/ForestCreatorFactory.cpp:7-11).
#pragma once
#include "forest.h"

#include <string>

namespace tb {

// Each returns an empty string on success, else the reason.
std::string load_xgboost_json(const std::string &path, Forest *out);
// num_features_hint: the caller's feature count (the reference requires it for ONNX,
// src/json/onnxmodelparser.h:334-337); the loader uses max(hint, largest feature id + 1).
std::string load_onnx_file(const std::string &path, int32_t num_features_hint, Forest *out);
std::string load_onnx_file(const std::string &path, Forest *out);

} // namespace tb
