// Model file front ends.  Names follow the reference's forest-creator factory
// ("xgboost_json", "onnx_file": src/json/ForestCreatorFactory.cpp:7-11).
#pragma once
#include "forest.h"

#include <string>

namespace tb {

// Each returns an empty string on success, else the reason.
std::string load_xgboost_json(const std::string &path, Forest *out);
std::string load_onnx_file(const std::string &path, Forest *out);

} // namespace tb
