// Compiled-model files: the forest in binary form plus the options a runner was built
// with, so that a later process can create the same runner without parsing the model's
// JSON / ONNX text again.
//
// The reference keeps a compiled model as two files -- a shared object with the generated
// code and a "globals" JSON that its serializer writes next to it (tile size, type widths,
// the packed buffers: src/utils/TreeTilingUtils.cpp:95-170) -- and reloads the pair with
// InitializeInferenceRunner(soPath, globalsJSONPath) (src/runtime/runtime.cpp:35-54).
// Here the pair is
//   * the MODEL FILE (binary, little endian): header, bound options, forest arrays in the
//     model's own node numbering (so leaf ids stay those of the model file), checksum; then,
//     optionally, the PACKED IMAGE of the forest (packed_image.h: the layout chosen for the
//     bound options and its buffers, ready for upload, with a checksum of its own), so that
//     loading skips the packer.  A loader that finds the image stale or damaged drops it and
//     packs the forest arrays again;
//   * the GLOBALS JSON (text): the bound options again, readable and editable; when it is
//     given to the loader its values replace those of the model file, which is how a tuned
//     launch shape or another batch size is applied without rewriting the binary.
#pragma once
#include "forest.h"

#include <cstdint>
#include <string>
#include <vector>

namespace tb {

// What build_runner() needs besides the forest.  Zero in a launch-shape field = "choose".
struct ModelFileOptions {
  int32_t batch_size = 0;
  int32_t tile_size = 1;
  int32_t threshold_width = 32, feature_index_width = 16, input_width = 32;
  int32_t return_width = 32, return_is_float = 1;
  int32_t number_of_features = 0;
  int32_t has_gpu_options = 0;
  int32_t rows_per_block = 0, rows_per_thread = 0, tree_threads = 0, cache_trees = 0, cache_rows = 0;
  std::string representation; // "gpu_sparse" | "gpu_array" | "gpu_reorg" | "" (process default)
};

constexpr uint32_t kModelFileVersion = 2;

// Each returns an empty string on success, else the reason.  `image`: the serialised packed
// image to append (may be null or empty) / where to put the one found (may be null; left
// empty when the file has none or its section is cut short).
std::string save_model_file(const std::string &path, const Forest &f, const ModelFileOptions &o,
                            const std::vector<uint8_t> *image = nullptr);
std::string load_model_file(const std::string &path, Forest *f, ModelFileOptions *o,
                            std::vector<uint8_t> *image = nullptr);

std::string save_globals_json(const std::string &path, const Forest &f, const ModelFileOptions &o);
// Overwrites the fields of *o that the JSON names.
std::string load_globals_json(const std::string &path, ModelFileOptions *o);

} // namespace tb
