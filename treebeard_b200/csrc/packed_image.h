// A packed forest as it lies in host memory just before the upload: the layout that was
// chosen for it (general tiles / 16-bit keys for wide rows / one tree per stage for deep
// trees) and that layout's buffers.  It can be serialised, which is what a compiled-model
// file caches so that loading it skips the packer -- the counterpart of the buffers the
// reference's serializer writes next to a compiled module and reloads
// (src/utils/TreeTilingUtils.cpp:95-170, src/runtime/runtime.cpp:35-54).
#pragma once
#include "../../include/tbk.h"
#include "deep_pack.h"
#include "pack.h"
#include "quant_pack.h"

#include <cstdint>
#include <string>
#include <vector>

namespace tb {

struct PackedImage {
  enum Kind : int32_t { kGeneral = 0, kQuant = 1, kDeep = 2 };
  int32_t kind = kGeneral;
  // what was asked for (the key under which a cached image may be reused) ...
  int32_t requested_representation = 0, requested_tile_size = 1, requested_feature_bits = 0;
  int32_t smem_limit = 0; // shared memory per block the layout was chosen for
  // ... and what was settled on
  tbk_schedule user{};
  int32_t deep_row_warps = 0, deep_slots = 0;
  PackedForest packed; // kGeneral
  QuantForest qf;      // kQuant
  DeepForest df;       // kDeep
};

constexpr uint32_t kPackedImageVersion = 6; // changes whenever a packer's output does

void serialize_image(const PackedImage &im, std::vector<uint8_t> *out);
uint64_t serialized_image_size(const PackedImage &im); // without serialising
// Empty string on success.  Checks the version, sizes and a checksum; a stale or damaged
// image is an error, never a partially filled structure.
std::string deserialize_image(const uint8_t *data, uint64_t size, PackedImage *im);

} // namespace tb
