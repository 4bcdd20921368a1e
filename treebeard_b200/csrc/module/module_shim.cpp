// The module-side symbols of the reference's inference runner (include/tbk_module.h): the
// buffers that the reference's serializers hand to Init_* are turned back into a forest, which
// is packed and uploaded through the kernel library (include/tbk.h) on the first prediction.
// Compiled twice: as is for the array / sparse serializers (libtbk_module.so), and with
// TBK_MODULE_REORG for the reorg serializer, whose Prediction_Function and Dealloc_Buffers
// carry other arguments under the same names (libtbk_module_reorg.so).
#include "../../../include/tbk_module.h"
#include "../../../include/tbk.h"

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

namespace {

struct Module {
  tbk_module_config cfg{};
  bool configured = false;
  std::vector<float> thr;
  std::vector<int32_t> feat, child;
  std::vector<int64_t> offsets, lengths;
  std::vector<int8_t> class_ids;
  tbk_forest *forest = nullptr;
  std::string error;
  std::mutex mu;
};

Module g;

int32_t fail(const char *fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g.error = buf;
  return 1;
}

tbk_memref1 memref(void *ptr, int64_t size) { return tbk_memref1{ptr, ptr, 0, {size}, {1}}; }

// element `i` of a strided index buffer of the given bit width
int32_t index_at(const void *aligned, int64_t offset, int64_t stride, int64_t i, int32_t width) {
  const int64_t k = offset + i * stride;
  if (width == 8) return static_cast<const int8_t *>(aligned)[k];
  if (width == 16) return static_cast<const int16_t *>(aligned)[k];
  return static_cast<const int32_t *>(aligned)[k];
}

void drop_forest() {
  if (g.forest) tbk_forest_free(g.forest);
  g.forest = nullptr;
}

// Flat forest arrays under construction: per tree the nodes reachable from slot 0 of the
// serialized tree, renumbered in the order they are met (the array layouts also hold slots
// that no walk reaches).
struct Rebuilt {
  std::vector<int64_t> tree_off{0};
  std::vector<int32_t> left, right, feat, cls;
  std::vector<float> thr;

  // `element(slot)` = index into g.thr / g.feat, `left_child(slot, element)` = slot of the left
  // child (the right child follows it), `slots` = slots the tree may use
  template <typename Element, typename LeftChild>
  int32_t add_tree(int64_t t, int64_t slots, Element element, LeftChild left_child) {
    const size_t base = left.size();
    std::vector<int64_t> kept{0}; // serialized slot of every node kept, in output order
    for (size_t k = 0; k < kept.size(); ++k) {
      const int64_t s = kept[k], e = element(s);
      const int32_t f = g.feat[e];
      thr.push_back(g.thr[e]);
      if (f < 0) { // a leaf: the value sits in the threshold
        feat.push_back(0);
        left.push_back(-1);
        right.push_back(-1);
        continue;
      }
      const int64_t l = left_child(s, e);
      if (l < 0 || l + 1 >= slots) return fail("tree %lld: child of slot %lld outside the tree", (long long)t, (long long)s);
      feat.push_back(f);
      left.push_back((int32_t)kept.size());
      right.push_back((int32_t)kept.size() + 1);
      kept.push_back(l);
      kept.push_back(l + 1);
      if (kept.size() > (size_t)slots + 2) return fail("tree %lld: the child links do not form a tree", (long long)t);
    }
    tree_off.push_back((int64_t)(base + kept.size()));
    cls.push_back(g.cfg.num_classes > 0 ? g.class_ids[t] : 0);
    return 0;
  }

  int32_t upload() {
    tbk_forest_arrays fa{};
    fa.num_trees = (int64_t)tree_off.size() - 1;
    fa.tree_off = tree_off.data();
    fa.left = left.data();
    fa.right = right.data();
    fa.feat = feat.data();
    fa.thr = thr.data();
    fa.class_id = g.cfg.num_classes > 0 ? cls.data() : nullptr;
    fa.num_classes = g.cfg.num_classes;
    fa.transform = g.cfg.transform;
    fa.initial_value = g.cfg.initial_value;
    fa.num_features = g.cfg.row_size;
    tbk_schedule sched{};
    sched.representation = TBK_REP_AUTO;
    drop_forest();
    if (tbk_forest_create(&fa, &sched, g.cfg.device, g.cfg.batch_size, &g.forest) != TBK_OK) return fail("%s", tbk_last_error());
    return 0;
  }
};

#ifndef TBK_MODULE_REORG
// array / sparse: every tree is a contiguous run [offset, offset + length) of the model buffer
int32_t build_forest() {
  const int64_t T = (int64_t)g.offsets.size();
  if (T == 0 || g.lengths.size() != (size_t)T) return fail("Init_Offsets / Init_Lengths have not both been called");
  if (g.thr.empty() || g.feat.size() != g.thr.size()) return fail("Init_Model has not been called");
  if (g.cfg.sparse && g.child.size() != g.thr.size()) return fail("the sparse representation needs child indices");
  if (g.cfg.num_classes > 0 && g.class_ids.size() != (size_t)T) return fail("Init_ClassIds has not been called");
  Rebuilt r;
  for (int64_t t = 0; t < T; ++t) {
    const int64_t off = g.offsets[t], len = g.lengths[t];
    if (off < 0 || len <= 0 || off + len > (int64_t)g.thr.size()) return fail("tree %lld: bad offset / length", (long long)t);
    const bool sparse = g.cfg.sparse != 0;
    if (r.add_tree(
            t, len, [&](int64_t s) { return off + s; },
            [&](int64_t s, int64_t e) { return sparse ? (int64_t)g.child[e] : 2 * s + 1; }) != 0)
      return 1;
  }
  return r.upload();
}
#else
// reorg: slot s of tree t sits at s * num_trees + t; every tree is a complete array of the
// deepest tree's size, slots a tree does not use hold feature index -1
int32_t build_forest() {
  const int64_t T = g.cfg.num_trees;
  if (T <= 0) return fail("the reorg representation needs num_trees in the configuration");
  if (g.thr.empty()) return fail("Init_Thresholds has not been called");
  if (g.feat.size() != g.thr.size()) return fail("Init_Thresholds / Init_FeatureIndices differ in length");
  if (g.cfg.num_classes > 0 && g.class_ids.size() != (size_t)T) return fail("Init_ClassIds has not been called");
  const int64_t n = (int64_t)g.thr.size();
  const int64_t slots = n / T;
  if (slots * T != n || ((slots + 1) & slots) != 0) return fail("buffer length %lld is not num_trees x (2^depth - 1)", (long long)n);
  Rebuilt r;
  for (int64_t t = 0; t < T; ++t)
    if (r.add_tree(
            t, slots, [&](int64_t s) { return s * T + t; }, [&](int64_t s, int64_t) { return 2 * s + 1; }) != 0)
      return 1;
  return r.upload();
}
#endif

// the common part of both flavours of Prediction_Function
tbk_memref1 predict(void *inAligned, int64_t inOffset, int64_t inRows, int64_t inCols, int64_t inStride0, int64_t inStride1,
                    void *out, void *outAligned, int64_t outOffset, int64_t outSize, int64_t outStride) {
  std::lock_guard<std::mutex> lock(g.mu);
  const tbk_memref1 result{out, outAligned, outOffset, {outSize}, {outStride}};
  if (!g.configured) {
    fail("TBK_Module_Configure has not been called");
    return result;
  }
  if (inCols != g.cfg.row_size || inStride1 != 1 || outStride != 1 || outSize < inRows || inStride0 < inCols) {
    fail("Prediction_Function: row-major fp32 rows of %d features and a dense result are expected", g.cfg.row_size);
    return result;
  }
  if (!g.forest && build_forest() != 0) return result;
  const bool int8_out = g.cfg.return_width == 8;
  const float *rows = static_cast<const float *>(inAligned) + inOffset;
  void *dst = int8_out ? static_cast<void *>(static_cast<int8_t *>(outAligned) + outOffset)
                       : static_cast<void *>(static_cast<float *>(outAligned) + outOffset);
  if (tbk_predict_host(g.forest, rows, inRows, inStride0, dst, int8_out ? TBK_OUT_I8 : TBK_OUT_F32) != TBK_OK)
    fail("%s", tbk_last_error());
  else
    g.error.clear();
  return result;
}

void forget_buffers() {
  std::lock_guard<std::mutex> lock(g.mu);
  drop_forest();
  g.thr.clear();
  g.feat.clear();
  g.child.clear();
  g.offsets.clear();
  g.lengths.clear();
  g.class_ids.clear();
}

} // namespace

extern "C" {

int32_t TBK_Module_Configure(const tbk_module_config *c) {
  std::lock_guard<std::mutex> lock(g.mu);
  if (!c) return fail("null configuration");
  if (c->batch_size <= 0 || c->row_size <= 0) return fail("batch size and row size must be positive");
  if (c->feature_index_width != 8 && c->feature_index_width != 16 && c->feature_index_width != 32)
    return fail("feature indices must be 8, 16 or 32 bits wide");
  if (c->sparse && c->child_index_width != 16 && c->child_index_width != 32) return fail("child indices must be 16 or 32 bits wide");
  if (c->return_width != 32 && !(c->return_width == 8 && c->num_classes > 0)) return fail("results are fp32 or (multiclass) int8");
  g.cfg = *c;
  g.configured = true;
  drop_forest();
  g.error.clear();
  return 0;
}

const char *TBK_Module_LastError(void) { return g.error.c_str(); }

int32_t GetBatchSize(void) { return g.cfg.batch_size; }
int32_t GetRowSize(void) { return g.cfg.row_size; }
int32_t GetInputTypeBitWidth(void) { return 32; }
int32_t GetReturnTypeBitWidth(void) { return g.cfg.return_width ? g.cfg.return_width : 32; }

tbk_memref1 Init_ClassIds(int8_t *, int8_t *aligned, int64_t offset, int64_t size, int64_t stride) {
  std::lock_guard<std::mutex> lock(g.mu);
  g.class_ids.resize(size > 0 ? size : 0);
  for (int64_t i = 0; i < size; ++i) g.class_ids[i] = aligned[offset + i * stride];
  drop_forest();
  return memref(g.class_ids.data(), size);
}

#ifndef TBK_MODULE_REORG

tbk_memref1 Init_Lengths(int64_t *, int64_t *aligned, int64_t offset, int64_t size, int64_t stride) {
  std::lock_guard<std::mutex> lock(g.mu);
  g.lengths.resize(size > 0 ? size : 0);
  for (int64_t i = 0; i < size; ++i) g.lengths[i] = aligned[offset + i * stride];
  drop_forest();
  return memref(g.lengths.data(), size);
}

tbk_memref1 Init_Offsets(int64_t *, int64_t *aligned, int64_t offset, int64_t size, int64_t stride) {
  std::lock_guard<std::mutex> lock(g.mu);
  g.offsets.resize(size > 0 ? size : 0);
  for (int64_t i = 0; i < size; ++i) g.offsets[i] = aligned[offset + i * stride];
  drop_forest();
  return memref(g.offsets.data(), size);
}

tbk_memref1 Init_Model(void *, void *thrAligned, int64_t thrOffset, int64_t thrSize, int64_t thrStride,
                       void *, void *featAligned, int64_t featOffset, int64_t featSize, int64_t featStride,
                       void *, void *, int64_t, int64_t, int64_t,
                       void *, void *childAligned, int64_t childOffset, int64_t childSize, int64_t childStride) {
  std::lock_guard<std::mutex> lock(g.mu);
  drop_forest();
  g.thr.clear();
  g.feat.clear();
  g.child.clear();
  if (!g.configured) {
    fail("TBK_Module_Configure has not been called");
    return memref(nullptr, 0);
  }
  if (thrSize <= 0 || featSize != thrSize || (g.cfg.sparse && childSize != thrSize)) {
    fail("Init_Model: the buffers differ in length");
    return memref(nullptr, 0);
  }
  g.thr.resize(thrSize);
  g.feat.resize(thrSize);
  const float *thr = static_cast<const float *>(thrAligned);
  for (int64_t i = 0; i < thrSize; ++i) {
    g.thr[i] = thr[thrOffset + i * thrStride];
    g.feat[i] = index_at(featAligned, featOffset, featStride, i, g.cfg.feature_index_width);
  }
  if (g.cfg.sparse) { // (the child-index arguments exist only in the sparse flavour of the call)
    g.child.resize(thrSize);
    for (int64_t i = 0; i < thrSize; ++i)
      g.child[i] = index_at(childAligned, childOffset, childStride, i, g.cfg.child_index_width);
  }
  return memref(&g, thrSize); // the "model" memref is opaque to the caller: it only travels back
}

tbk_memref1 Prediction_Function(void *, void *inAligned, int64_t inOffset, int64_t inRows, int64_t inCols, int64_t inStride0,
                                int64_t inStride1, void *out, void *outAligned, int64_t outOffset, int64_t outSize,
                                int64_t outStride, void *, void *, int64_t, int64_t, int64_t, int64_t *, int64_t *, int64_t,
                                int64_t, int64_t, int64_t *, int64_t *, int64_t, int64_t, int64_t, int8_t *, int8_t *,
                                int64_t, int64_t, int64_t) {
  return predict(inAligned, inOffset, inRows, inCols, inStride0, inStride1, out, outAligned, outOffset, outSize, outStride);
}

int32_t Dealloc_Buffers(void *, void *, int64_t, int64_t, int64_t, int64_t *, int64_t *, int64_t, int64_t, int64_t,
                        int64_t *, int64_t *, int64_t, int64_t, int64_t) {
  forget_buffers();
  return 0;
}

#else // TBK_MODULE_REORG

tbk_memref1 Init_Thresholds(float *, float *aligned, int64_t offset, int64_t size, int64_t stride) {
  std::lock_guard<std::mutex> lock(g.mu);
  drop_forest();
  g.thr.resize(size > 0 ? size : 0);
  for (int64_t i = 0; i < size; ++i) g.thr[i] = aligned[offset + i * stride];
  return memref(g.thr.data(), size);
}

tbk_memref1 Init_FeatureIndices(void *, void *aligned, int64_t offset, int64_t size, int64_t stride) {
  std::lock_guard<std::mutex> lock(g.mu);
  drop_forest();
  g.feat.clear();
  if (!g.configured) {
    fail("TBK_Module_Configure has not been called");
    return memref(nullptr, 0);
  }
  g.feat.resize(size > 0 ? size : 0);
  for (int64_t i = 0; i < size; ++i) g.feat[i] = index_at(aligned, offset, stride, i, g.cfg.feature_index_width);
  return memref(g.feat.data(), size);
}

tbk_memref1 Prediction_Function(void *, void *inAligned, int64_t inOffset, int64_t inRows, int64_t inCols, int64_t inStride0,
                                int64_t inStride1, void *out, void *outAligned, int64_t outOffset, int64_t outSize,
                                int64_t outStride, void *, void *, int64_t, int64_t, int64_t, void *, void *, int64_t, int64_t,
                                int64_t, int8_t *, int8_t *, int64_t, int64_t, int64_t) {
  return predict(inAligned, inOffset, inRows, inCols, inStride0, inStride1, out, outAligned, outOffset, outSize, outStride);
}

// (a multiclass module is also handed the class-id memref: five more arguments, not read)
int32_t Dealloc_Buffers(void *, void *, int64_t, int64_t, int64_t, void *, void *, int64_t, int64_t, int64_t) {
  forget_buffers();
  return 0;
}

#endif

} // extern "C"
