#include "packed_image.h"
#include "checksum.h"

#include <cstring>
#include <type_traits>

namespace tb {

namespace {

const char kImageMagic[8] = {'T', 'B', 'B', '2', 'I', 'M', 'G', '\0'};

uint64_t checksum(const uint8_t *p, size_t n) { return hash_bytes(kHashSeed, p, n); }

struct Out {
  std::vector<uint8_t> *b; // null: only count the bytes
  uint64_t count = 0;
  void raw(const void *p, size_t n) {
    count += n;
    if (!b) return;
    const uint8_t *c = static_cast<const uint8_t *>(p);
    b->insert(b->end(), c, c + n);
  }
  template <typename T> void pod(const T &v) {
    static_assert(std::is_trivially_copyable<T>::value, "plain data only");
    raw(&v, sizeof(T));
  }
  template <typename T> void vec(const std::vector<T> &v) {
    pod<uint64_t>(v.size());
    if (!v.empty()) raw(v.data(), v.size() * sizeof(T));
  }
};

struct In {
  const uint8_t *p;
  uint64_t left;
  bool ok = true;
  void raw(void *dst, size_t n) {
    if (!ok || n > left) {
      ok = false;
      return;
    }
    std::memcpy(dst, p, n);
    p += n;
    left -= n;
  }
  template <typename T> T pod() {
    T v{};
    raw(&v, sizeof(T));
    return v;
  }
  template <typename T> void vec(std::vector<T> *v) {
    const uint64_t n = pod<uint64_t>();
    if (!ok || n > left / sizeof(T)) { // a count larger than what is left is a damaged image
      ok = false;
      return;
    }
    v->resize(n);
    if (n) raw(v->data(), n * sizeof(T));
  }
};

void put_key_forest_head(Out &o, int32_t num_features, int32_t transform, double initial_value, int64_t num_trees,
                         int64_t num_nodes, int32_t max_depth) {
  o.pod(num_features);
  o.pod(transform);
  o.pod(initial_value);
  o.pod(num_trees);
  o.pod(num_nodes);
  o.pod(max_depth);
}

} // namespace

namespace {
void put_image(const PackedImage &im, Out &o) {
  o.raw(kImageMagic, sizeof(kImageMagic));
  o.pod<uint32_t>(kPackedImageVersion);
  o.pod(im.kind);
  o.pod(im.requested_representation);
  o.pod(im.requested_tile_size);
  o.pod(im.requested_feature_bits);
  o.pod(im.smem_limit);
  o.pod(im.user);
  o.pod(im.deep_row_warps);
  o.pod(im.deep_slots);
  if (im.kind == PackedImage::kGeneral) {
    const PackedForest &p = im.packed;
    o.pod(p.representation);
    o.pod(p.tile_size);
    o.pod(p.tile_bytes);
    o.pod(p.num_features);
    o.pod(p.num_classes);
    o.pod(p.transform);
    o.pod(p.initial_value);
    o.pod(p.num_trees);
    o.pod(p.num_nodes);
    o.pod(p.max_depth);
    o.pod(p.max_group_bytes);
    o.pod(p.num_shapes);
    o.vec(p.groups);
    o.vec(p.blob);
    o.vec(p.tree_class);
    o.vec(p.tree_index);
    o.vec(p.orig_off);
    o.vec(p.orig_node);
    o.vec(p.lut);
  } else if (im.kind == PackedImage::kQuant) {
    const QuantForest &q = im.qf;
    put_key_forest_head(o, q.num_features, q.transform, q.initial_value, q.num_trees, q.num_nodes, q.max_depth);
    o.vec(q.groups);
    o.vec(q.node_plane);
    o.vec(q.leaf_plane);
    o.vec(q.exact_plane);
    o.vec(q.orig_leaf);
    o.vec(q.tree_index);
    o.vec(q.lo);
    o.vec(q.scale);
    o.pod(q.num_classes);
    o.vec(q.group_class);
  } else {
    const DeepForest &q = im.df;
    put_key_forest_head(o, q.num_features, q.transform, q.initial_value, q.num_trees, q.num_nodes, q.max_depth);
    o.vec(q.pairs);
    o.vec(q.node_plane);
    o.vec(q.leaf_plane);
    o.vec(q.exact_plane);
    o.vec(q.orig_leaf);
    o.vec(q.tree_index);
    o.vec(q.lo);
    o.vec(q.scale);
  }
}
} // namespace

uint64_t serialized_image_size(const PackedImage &im) {
  Out o{nullptr};
  put_image(im, o);
  return o.count + 8;
}

void serialize_image(const PackedImage &im, std::vector<uint8_t> *out) {
  out->clear();
  out->reserve(serialized_image_size(im));
  Out o{out};
  put_image(im, o);
  const uint64_t sum = checksum(out->data(), out->size());
  o.pod(sum);
}

std::string deserialize_image(const uint8_t *data, uint64_t size, PackedImage *im) {
  if (size < sizeof(kImageMagic) + 4 + 8) return "packed image: too short";
  uint64_t sum = 0;
  std::memcpy(&sum, data + size - 8, 8);
  if (sum != checksum(data, size - 8)) return "packed image: checksum mismatch";
  In in{data, size - 8};
  char magic[sizeof(kImageMagic)];
  in.raw(magic, sizeof(magic));
  if (!in.ok || std::memcmp(magic, kImageMagic, sizeof(magic)) != 0) return "packed image: bad magic";
  const uint32_t version = in.pod<uint32_t>();
  if (version != kPackedImageVersion) return "packed image: version " + std::to_string(version) + " is not this library's";
  *im = PackedImage();
  im->kind = in.pod<int32_t>();
  im->requested_representation = in.pod<int32_t>();
  im->requested_tile_size = in.pod<int32_t>();
  im->requested_feature_bits = in.pod<int32_t>();
  im->smem_limit = in.pod<int32_t>();
  im->user = in.pod<tbk_schedule>();
  im->deep_row_warps = in.pod<int32_t>();
  im->deep_slots = in.pod<int32_t>();
  auto key_head = [&](int32_t *nf, int32_t *tr, double *iv, int64_t *nt, int64_t *nn, int32_t *md) {
    *nf = in.pod<int32_t>();
    *tr = in.pod<int32_t>();
    *iv = in.pod<double>();
    *nt = in.pod<int64_t>();
    *nn = in.pod<int64_t>();
    *md = in.pod<int32_t>();
  };
  if (im->kind == PackedImage::kGeneral) {
    PackedForest &p = im->packed;
    p.representation = in.pod<int32_t>();
    p.tile_size = in.pod<int32_t>();
    p.tile_bytes = in.pod<int32_t>();
    p.num_features = in.pod<int32_t>();
    p.num_classes = in.pod<int32_t>();
    p.transform = in.pod<int32_t>();
    p.initial_value = in.pod<double>();
    p.num_trees = in.pod<int64_t>();
    p.num_nodes = in.pod<int64_t>();
    p.max_depth = in.pod<int32_t>();
    p.max_group_bytes = in.pod<uint64_t>();
    p.num_shapes = in.pod<int32_t>();
    in.vec(&p.groups);
    in.vec(&p.blob);
    in.vec(&p.tree_class);
    in.vec(&p.tree_index);
    in.vec(&p.orig_off);
    in.vec(&p.orig_node);
    in.vec(&p.lut);
    if (in.ok && (p.tree_class.size() != p.groups.size() * kGroupTrees || p.tree_index.size() != p.tree_class.size() ||
                  p.orig_off.size() != p.groups.size()))
      in.ok = false;
    for (const GroupMeta &g : p.groups) // every group must lie inside the blob
      if (in.ok && g.byte_off + (uint64_t)g.slots * kGroupTrees * (p.representation == kReorg ? 6 : p.tile_bytes) > p.blob.size() + 15)
        in.ok = false;
  } else if (im->kind == PackedImage::kQuant) {
    QuantForest &q = im->qf;
    key_head(&q.num_features, &q.transform, &q.initial_value, &q.num_trees, &q.num_nodes, &q.max_depth);
    in.vec(&q.groups);
    in.vec(&q.node_plane);
    in.vec(&q.leaf_plane);
    in.vec(&q.exact_plane);
    in.vec(&q.orig_leaf);
    in.vec(&q.tree_index);
    in.vec(&q.lo);
    in.vec(&q.scale);
    q.num_classes = in.pod<int32_t>();
    in.vec(&q.group_class);
    const size_t n = q.node_plane.size();
    if (in.ok && (q.leaf_plane.size() != n || q.exact_plane.size() != n || q.orig_leaf.size() != n ||
                  q.tree_index.size() != q.groups.size() * kQuantCols || q.lo.size() != (size_t)q.num_features + 1 ||
                  q.scale.size() != q.lo.size() || q.num_classes < 0 ||
                  q.group_class.size() != (q.num_classes > 0 ? q.groups.size() : 0)))
      in.ok = false;
    for (const int32_t cls : q.group_class)
      if (cls < 0 || cls >= q.num_classes) in.ok = false;
    for (const QuantGroup &g : q.groups)
      if (in.ok && (g.depth < 1 || g.depth > (uint32_t)kQuantMaxDepth || g.slots != (1u << g.depth) ||
                    g.elem_off + (uint64_t)g.slots * kQuantCols > n))
        in.ok = false;
  } else if (im->kind == PackedImage::kDeep) {
    DeepForest &q = im->df;
    key_head(&q.num_features, &q.transform, &q.initial_value, &q.num_trees, &q.num_nodes, &q.max_depth);
    in.vec(&q.pairs);
    in.vec(&q.node_plane);
    in.vec(&q.leaf_plane);
    in.vec(&q.exact_plane);
    in.vec(&q.orig_leaf);
    in.vec(&q.tree_index);
    in.vec(&q.lo);
    in.vec(&q.scale);
    const size_t n = q.node_plane.size();
    if (in.ok && (q.leaf_plane.size() != n || q.exact_plane.size() != n || q.orig_leaf.size() != n ||
                  q.tree_index.size() != q.pairs.size() * 2 || q.lo.size() != (size_t)q.num_features + 1 ||
                  q.scale.size() != q.lo.size()))
      in.ok = false;
    for (const QuantGroup &g : q.pairs)
      if (in.ok && (g.depth > (uint32_t)kDeepMaxDepth || g.elem_off + 2ull * g.slots > n)) in.ok = false;
  } else {
    return "packed image: unknown layout kind";
  }
  if (!in.ok || in.left != 0) return "packed image: truncated or inconsistent";
  return "";
}

} // namespace tb
