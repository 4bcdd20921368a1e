#include "model_file.h"
#include "checksum.h"
#include "json.h"

#include <cstdio>
#include <cstring>
#include <fstream>
#include <sstream>
#include <vector>

namespace tb {

namespace {

const char kMagic[8] = {'T', 'B', 'B', '2', 'M', 'D', 'L', '\0'};
const char kImageSection[8] = {'T', 'B', 'B', '2', 'S', 'E', 'C', '1'}; // opens the optional packed-image section

// checksum over the payload, chunk by chunk as it is written (checksum.h)
uint64_t checksum(uint64_t h, const void *data, size_t n) { return hash_bytes(h, data, n); }

struct Writer {
  std::FILE *fp;
  uint64_t hash = 14695981039346656037ull;
  bool ok = true;
  void raw(const void *p, size_t n) {
    if (n == 0) return;
    if (std::fwrite(p, 1, n, fp) != n) ok = false;
    hash = checksum(hash, p, n);
  }
  template <typename T> void pod(const T &v) { raw(&v, sizeof(T)); }
  template <typename T> void vec(const std::vector<T> &v) {
    pod<uint64_t>(v.size());
    raw(v.data(), v.size() * sizeof(T));
  }
  void str(const std::string &s) {
    pod<uint64_t>(s.size());
    raw(s.data(), s.size());
  }
};

struct Reader {
  std::FILE *fp;
  uint64_t hash = 14695981039346656037ull;
  uint64_t remaining;
  bool ok = true;
  void raw(void *p, size_t n) {
    if (!ok || n == 0) return;
    if (n > remaining || std::fread(p, 1, n, fp) != n) {
      ok = false;
      return;
    }
    remaining -= n;
    hash = checksum(hash, p, n);
  }
  template <typename T> T pod() {
    T v{};
    raw(&v, sizeof(T));
    return v;
  }
  template <typename T> void vec(std::vector<T> *v) {
    const uint64_t n = pod<uint64_t>();
    if (!ok || n > remaining / sizeof(T)) { // a count larger than the file is a corrupt file
      ok = false;
      return;
    }
    v->resize(n);
    raw(v->data(), n * sizeof(T));
  }
  void str(std::string *s) {
    const uint64_t n = pod<uint64_t>();
    if (!ok || n > remaining || n > (1u << 20)) {
      ok = false;
      return;
    }
    s->resize(n);
    raw(&(*s)[0], n);
  }
};

const int kOptionInts = 14;
void options_to_ints(const ModelFileOptions &o, int32_t *v) {
  const int32_t src[kOptionInts] = {o.batch_size, o.tile_size, o.threshold_width, o.feature_index_width,
                                    o.input_width, o.return_width, o.return_is_float, o.number_of_features,
                                    o.has_gpu_options, o.rows_per_block, o.rows_per_thread, o.tree_threads,
                                    o.cache_trees, o.cache_rows};
  std::memcpy(v, src, sizeof(src));
}
void ints_to_options(const int32_t *v, ModelFileOptions *o) {
  o->batch_size = v[0];
  o->tile_size = v[1];
  o->threshold_width = v[2];
  o->feature_index_width = v[3];
  o->input_width = v[4];
  o->return_width = v[5];
  o->return_is_float = v[6];
  o->number_of_features = v[7];
  o->has_gpu_options = v[8];
  o->rows_per_block = v[9];
  o->rows_per_thread = v[10];
  o->tree_threads = v[11];
  o->cache_trees = v[12];
  o->cache_rows = v[13];
}

} // namespace

std::string save_model_file(const std::string &path, const Forest &f, const ModelFileOptions &o,
                            const std::vector<uint8_t> *image) {
  std::string err = validate(f);
  if (!err.empty()) return err;
  std::FILE *fp = std::fopen(path.c_str(), "wb");
  if (!fp) return "cannot open \"" + path + "\" for writing";
  Writer w{fp};
  w.raw(kMagic, sizeof(kMagic));
  w.pod<uint32_t>(kModelFileVersion);
  w.pod<uint32_t>(kOptionInts);
  int32_t ints[kOptionInts];
  options_to_ints(o, ints);
  w.raw(ints, sizeof(ints));
  w.str(o.representation);
  w.pod<int32_t>(f.num_classes);
  w.pod<int32_t>(f.transform);
  w.pod<int32_t>(f.num_features);
  w.pod<double>(f.initial_value);
  w.vec(f.tree_off);
  w.vec(f.left);
  w.vec(f.right);
  w.vec(f.feat);
  w.vec(f.thr);
  w.vec(f.class_id);
  const uint64_t sum = w.hash;
  if (std::fwrite(&sum, 1, sizeof(sum), fp) != sizeof(sum)) w.ok = false;
  if (image && !image->empty()) { // after the checksum: a damaged image must not spoil the forest
    const uint64_t n = image->size();
    if (std::fwrite(kImageSection, 1, sizeof(kImageSection), fp) != sizeof(kImageSection) ||
        std::fwrite(&n, 1, sizeof(n), fp) != sizeof(n) || std::fwrite(image->data(), 1, n, fp) != n)
      w.ok = false;
  }
  if (std::fclose(fp) != 0) w.ok = false;
  if (!w.ok) {
    std::remove(path.c_str());
    return "write to \"" + path + "\" failed";
  }
  return "";
}

std::string load_model_file(const std::string &path, Forest *f, ModelFileOptions *o, std::vector<uint8_t> *image) {
  if (image) image->clear();
  std::FILE *fp = std::fopen(path.c_str(), "rb");
  if (!fp) return "cannot open \"" + path + "\"";
  std::fseek(fp, 0, SEEK_END);
  const long size = std::ftell(fp);
  std::fseek(fp, 0, SEEK_SET);
  if (size < (long)(sizeof(kMagic) + 16)) {
    std::fclose(fp);
    return "\"" + path + "\" is not a compiled-model file (too short)";
  }
  Reader r{fp};
  r.remaining = (uint64_t)size; // (the checksum trails the payload; an image section may follow it)
  char magic[sizeof(kMagic)];
  r.raw(magic, sizeof(magic));
  if (!r.ok || std::memcmp(magic, kMagic, sizeof(kMagic)) != 0) {
    std::fclose(fp);
    return "\"" + path + "\" is not a compiled-model file (bad magic)";
  }
  const uint32_t version = r.pod<uint32_t>();
  const uint32_t n_ints = r.pod<uint32_t>();
  if (!r.ok || version != kModelFileVersion || n_ints != (uint32_t)kOptionInts) {
    std::fclose(fp);
    return "\"" + path + "\": unsupported compiled-model file version " + std::to_string(version);
  }
  int32_t ints[kOptionInts];
  r.raw(ints, sizeof(ints));
  ints_to_options(ints, o);
  r.str(&o->representation);
  *f = Forest();
  f->num_classes = r.pod<int32_t>();
  f->transform = r.pod<int32_t>();
  f->num_features = r.pod<int32_t>();
  f->initial_value = r.pod<double>();
  r.vec(&f->tree_off);
  r.vec(&f->left);
  r.vec(&f->right);
  r.vec(&f->feat);
  r.vec(&f->thr);
  r.vec(&f->class_id);
  uint64_t sum = 0;
  bool tail = r.ok && r.remaining >= sizeof(sum) && std::fread(&sum, 1, sizeof(sum), fp) == sizeof(sum);
  uint64_t rest = tail ? r.remaining - sizeof(sum) : 0;
  if (tail && rest > 0) {
    // only a packed-image section may follow; a section that is cut short is dropped (the
    // forest arrays above are complete), anything else is a damaged file
    char tag[sizeof(kImageSection)];
    uint64_t n = 0;
    if (rest < sizeof(tag) + sizeof(n) || std::fread(tag, 1, sizeof(tag), fp) != sizeof(tag) ||
        std::memcmp(tag, kImageSection, sizeof(tag)) != 0 || std::fread(&n, 1, sizeof(n), fp) != sizeof(n)) {
      tail = false;
    } else {
      rest -= sizeof(tag) + sizeof(n);
      if (n == rest && image) {
        image->resize(n);
        if (std::fread(image->data(), 1, n, fp) != n) image->clear();
      } else if (n < rest) {
        tail = false; // bytes behind the section
      }
    }
  }
  std::fclose(fp);
  if (!tail) return "\"" + path + "\" is truncated or has trailing bytes";
  if (sum != r.hash) return "\"" + path + "\": checksum mismatch";
  if (f->tree_off.empty()) return "\"" + path + "\": empty forest";
  return validate(*f);
}

std::string save_globals_json(const std::string &path, const Forest &f, const ModelFileOptions &o) {
  std::ofstream out(path);
  if (!out) return "cannot open \"" + path + "\" for writing";
  // "TileSizeEntries" keeps the shape of the reference's globals file
  // (src/runtime/runtime.cpp:43-48 reads TileSize / ThresholdBitWidth / FeatureIndexBitWidth)
  out << "{\n"
      << "  \"Format\": \"treebeard-b200-globals\",\n"
      << "  \"Version\": " << kModelFileVersion << ",\n"
      << "  \"TileSizeEntries\": [{\"TileSize\": " << o.tile_size << ", \"ThresholdBitWidth\": " << o.threshold_width
      << ", \"FeatureIndexBitWidth\": " << o.feature_index_width << "}],\n"
      << "  \"BatchSize\": " << o.batch_size << ",\n"
      << "  \"RowSize\": " << (o.number_of_features > f.num_features ? o.number_of_features : f.num_features) << ",\n"
      << "  \"InputElementBitWidth\": " << o.input_width << ",\n"
      << "  \"ReturnTypeBitWidth\": " << o.return_width << ",\n"
      << "  \"ReturnTypeIsFloat\": " << (o.return_is_float ? "true" : "false") << ",\n"
      << "  \"Representation\": \"" << o.representation << "\",\n"
      << "  \"NumberOfTrees\": " << f.num_trees() << ",\n"
      << "  \"NumberOfClasses\": " << f.num_classes << ",\n"
      << "  \"GPUSchedule\": {\"Pinned\": " << (o.has_gpu_options ? "true" : "false")
      << ", \"NumRowsPerTB\": " << o.rows_per_block << ", \"NumRowsPerThread\": " << o.rows_per_thread
      << ", \"NumTreeThreads\": " << o.tree_threads << ", \"CacheTrees\": " << (o.cache_trees ? "true" : "false")
      << ", \"CacheRows\": " << (o.cache_rows ? "true" : "false") << "}\n"
      << "}\n";
  out.close();
  return out ? "" : "write to \"" + path + "\" failed";
}

std::string load_globals_json(const std::string &path, ModelFileOptions *o) {
  std::ifstream in(path, std::ios::binary);
  if (!in) return "cannot open \"" + path + "\"";
  std::stringstream ss;
  ss << in.rdbuf();
  const std::string text = ss.str();
  try {
    json::Parser parser(text.data(), text.data() + text.size());
    const json::Value root = parser.parse();
    if (!root.is_object()) return "\"" + path + "\": globals JSON is not an object";
    if (root.has("TileSizeEntries")) {
      const json::Array &entries = root.at("TileSizeEntries").array();
      if (entries.size() != 1) return "\"" + path + "\": exactly one tile-size entry is expected";
      const json::Value &e = entries.front();
      if (e.has("TileSize")) o->tile_size = (int32_t)e.at("TileSize").number();
      if (e.has("ThresholdBitWidth")) o->threshold_width = (int32_t)e.at("ThresholdBitWidth").number();
      if (e.has("FeatureIndexBitWidth")) o->feature_index_width = (int32_t)e.at("FeatureIndexBitWidth").number();
    }
    if (root.has("BatchSize")) o->batch_size = (int32_t)root.at("BatchSize").number();
    if (root.has("InputElementBitWidth")) o->input_width = (int32_t)root.at("InputElementBitWidth").number();
    if (root.has("ReturnTypeBitWidth")) o->return_width = (int32_t)root.at("ReturnTypeBitWidth").number();
    if (root.has("ReturnTypeIsFloat")) o->return_is_float = root.at("ReturnTypeIsFloat").number() != 0.0;
    if (root.has("Representation")) o->representation = root.at("Representation").string();
    if (root.has("GPUSchedule")) {
      const json::Value &g = root.at("GPUSchedule");
      if (g.has("Pinned")) o->has_gpu_options = g.at("Pinned").number() != 0.0;
      if (g.has("NumRowsPerTB")) o->rows_per_block = (int32_t)g.at("NumRowsPerTB").number();
      if (g.has("NumRowsPerThread")) o->rows_per_thread = (int32_t)g.at("NumRowsPerThread").number();
      if (g.has("NumTreeThreads")) o->tree_threads = (int32_t)g.at("NumTreeThreads").number();
      if (g.has("CacheTrees")) o->cache_trees = g.at("CacheTrees").number() != 0.0;
      if (g.has("CacheRows")) o->cache_rows = g.at("CacheRows").number() != 0.0;
    }
  } catch (const std::exception &e) {
    return "\"" + path + "\": " + e.what();
  }
  return "";
}

} // namespace tb
