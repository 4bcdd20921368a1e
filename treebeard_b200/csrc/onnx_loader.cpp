// ONNX TreeEnsembleRegressor / TreeEnsembleClassifier -> Forest.
#include "loaders.h"

namespace tb {

std::string load_onnx_file(const std::string &path, Forest *) {
  return "ONNX models are not supported yet (" + path + ")";
}

} // namespace tb
