// The compile-then-run inference-runner API (see include/tbruntime.h), implemented over
// the kernel library's C ABI (include/tbk.h).  "Compiling" a model here means: load the
// model file into the host forest (front end), pack it in the chosen representation and
// upload it, and bind the launch-shape options; "running" dispatches the walk kernels.
// Reference: src/runtime/runtime.cpp (entry points), src/mlir/ExecutionHelpers.{h,cpp}
// and src/gpu/GPUExecutionHelper.{h,cpp} (runner objects).
#include "../../include/tbruntime.h"
#include "../../include/tbk.h"
#include "forest.h"
#include "loaders.h"
#include "model_file.h"

#include <cuda_runtime_api.h>

#include <cstdio>
#include <cstring>
#include <memory>
#include <mutex>
#include <thread>
#include <set>
#include <sstream>
#include <string>
#include <vector>

namespace {

thread_local int32_t g_status = 0;
thread_local std::string g_error;
int32_t g_device = 0;
std::vector<int32_t> g_more_devices; // further devices of the next runner (TB_SetDevices)
bool g_use_sparse = false;  // process-wide default representation (src/mlir/Dialect.cpp:104-110)
bool g_rep_flag_set = false; // ... once SetEnableSparseRepresentation has been called; until then the library chooses
bool g_peeled_codegen = false;
bool g_measure_kernel_time = false;
int32_t g_kernel_runs = 1;

void set_error(int32_t status, const std::string &msg) {
  g_status = status;
  g_error = msg;
}
void clear_error() {
  g_status = 0;
  g_error.clear();
}

// src/include/TreebeardContext.h:64-136
struct CompilerOptions {
  int32_t numberOfFeatures = -1;
  int32_t batchSize = 0;
  int32_t tileSize = 1;
  int32_t thresholdTypeWidth = 32;
  int32_t returnTypeWidth = 32;
  bool returnTypeFloatType = true;
  int32_t featureIndexTypeWidth = 16;
  int32_t nodeIndexTypeWidth = 16;
  int32_t inputElementTypeWidth = 32;
  int32_t tileShapeBitWidth = 16;
  int32_t childIndexBitWidth = 16;
  int32_t tilingType = 0;
  bool makeAllLeavesSameDepth = false;
  bool reorderTreesByDepth = false;
  int32_t pipelineSize = -1;
  std::string statsProfileCSVPath;
  int32_t numberOfCores = -1;
  int32_t numParallelTreeBatches = -1;
  bool oneTreeAtATime = false;
};

// src/include/TreebeardContext.h:138-162
struct GPUAutoScheduleOptions {
  int32_t numRowsPerTB = 0;
  int32_t numRowsPerThread = 0;
  int32_t rowTileSize = 0;
  int32_t numTreeThreads = 0;
  int32_t numTreesAtATime = 0;
  bool cacheRows = false;
  bool cacheTrees = false;
  bool unrollTreeWalks = false;
  int32_t treeWalkInterleaveFactor = -1;
  bool sharedMemoryReduce = false;
};

struct Schedule;
struct IndexVariable {
  std::string name;
  Schedule *owner = nullptr;
  int32_t gpuConstruct = -1, gpuDim = -1;
};

// Loop-nest description object.  The kernels implement one fixed loop nest, so
// directives are only recorded (and printed); see include/tbruntime.h.
struct Schedule {
  int32_t batchSize = 0, forestSize = 0;
  std::vector<std::unique_ptr<IndexVariable>> vars;
  IndexVariable *batch = nullptr, *tree = nullptr;
  std::vector<std::string> directives;
  bool touched = false;
  Schedule(int32_t b, int32_t t) : batchSize(b), forestSize(t) {
    batch = add("batch");
    tree = add("tree");
  }
  IndexVariable *add(const std::string &n) {
    vars.emplace_back(new IndexVariable{n, this});
    return vars.back().get();
  }
  void note(const std::string &d) {
    directives.push_back(d);
    touched = true;
  }
};

struct TreebeardContext {
  std::string modelPath, globalsPath;
  CompilerOptions options;
  bool hasGpuOptions = false;
  GPUAutoScheduleOptions gpuOptions;
  std::string creatorType = "xgboost_json";
  std::string representation; // empty: process default
  tb::Forest forest;
  bool forestLoaded = false;
  std::unique_ptr<Schedule> schedule;
};

struct InferenceRunner {
  tbk_forest *forest = nullptr;
  int32_t batchSize = 0, rowSize = 0;
  int32_t inputWidth = 32, returnWidth = 32;
  bool returnFloat = true;
  int32_t numClasses = 0;
  int32_t device = 0;
  // a runner over several devices: one more copy of the forest per further device; host batches
  // are cut into one contiguous row range per device and predicted concurrently
  std::vector<tbk_forest *> moreForests;
  std::vector<int32_t> moreDevices;
  bool fromPackedImage = false; // built from the packed image of a compiled-model file
  int64_t kernelMicros = 0;
};

std::mutex g_live_mu;
std::set<void *> g_representations;

const char *name_of(const IndexVariable *v) { return v ? v->name.c_str() : "?"; }

int rep_from_name(const std::string &name) {
  if (name == "gpu_array" || name == "array") return TBK_REP_ARRAY;
  if (name == "gpu_sparse" || name == "sparse") return TBK_REP_SPARSE;
  if (name == "gpu_reorg") return TBK_REP_REORG;
  if (name == "gpu_auto") return TBK_REP_AUTO; // addition: the library picks the layout
  return -2;
}

bool load_forest(const std::string &creator, const std::string &path, tb::Forest *f, int32_t num_features = 0) {
  std::string err;
  if (creator == "xgboost_json") err = tb::load_xgboost_json(path, f);
  else if (creator == "onnx_file") err = tb::load_onnx_file(path, num_features, f);
  else if (creator == "compiled_model") { // host-side readers only (TB_LoadForest)
    tb::ModelFileOptions ignored;
    err = tb::load_model_file(path, f, &ignored);
  }
  else err = "unknown forest creator \"" + creator + "\"";
  if (!err.empty()) {
    set_error(TBK_ERR_IO, err);
    return false;
  }
  return true;
}

// cached_image: serialised packed image found in a compiled-model file (may be null).
// save_image: when given, nothing is uploaded: the forest is packed for these options and the
// serialised image is left there (the return value is null; failures are in the error state).
InferenceRunner *build_runner(const tb::Forest &forest, const CompilerOptions &opt,
                              const GPUAutoScheduleOptions *gpu, const std::string &repName,
                              const std::vector<uint8_t> *cached_image = nullptr,
                              std::vector<uint8_t> *save_image = nullptr) {
  if (opt.batchSize <= 0) {
    set_error(TBK_ERR_INVALID, "batch size must be positive");
    return nullptr;
  }
  // 64-bit types (the reference's other tested combination, f64 thresholds / i32 indices): the
  // walk computes in fp32 either way -- thresholds of the supported model formats are fp32
  // values --; a 64-bit input or return width means that the HOST buffers of RunInference hold
  // doubles, converted on the way in and out.  Index widths do not matter to this library.
  if ((opt.thresholdTypeWidth != 32 && opt.thresholdTypeWidth != 64) ||
      (opt.inputElementTypeWidth != 32 && opt.inputElementTypeWidth != 64)) {
    set_error(TBK_ERR_UNSUPPORTED, "thresholds and inputs must be 32 or 64 bits wide");
    return nullptr;
  }
  if (opt.tilingType != 0) {
    set_error(TBK_ERR_UNSUPPORTED, "only uniform tiling is supported on the GPU path");
    return nullptr;
  }
  const bool int8_out = !opt.returnTypeFloatType && opt.returnTypeWidth == 8;
  if (!int8_out && !(opt.returnTypeFloatType && (opt.returnTypeWidth == 32 || opt.returnTypeWidth == 64))) {
    set_error(TBK_ERR_UNSUPPORTED, "return type must be fp32, fp64 or (multiclass) int8");
    return nullptr;
  }
  if (int8_out && forest.num_classes == 0) {
    set_error(TBK_ERR_INVALID, "int8 return type needs a multiclass model");
    return nullptr;
  }
  // no representation named and the sparse switch never touched: the library's own choice
  // (every layout selects the same leaves; the reference's array default is a code-generation detail)
  int rep = !repName.empty() ? rep_from_name(repName) : !g_rep_flag_set ? TBK_REP_AUTO : g_use_sparse ? TBK_REP_SPARSE : TBK_REP_ARRAY;
  if (rep < TBK_REP_AUTO) {
    set_error(TBK_ERR_INVALID, "unknown representation \"" + repName + "\"");
    return nullptr;
  }
  tbk_schedule sched{};
  sched.representation = rep;
  sched.tile_size = opt.tileSize <= 0 ? 1 : opt.tileSize;
  if (gpu) {
    sched.rows_per_block = gpu->numRowsPerTB;
    sched.rows_per_thread = gpu->numRowsPerThread;
    sched.tree_threads = gpu->numTreeThreads;
    sched.cache_trees = gpu->cacheTrees ? 1 : 0;
  }
  tbk_forest_arrays fa{};
  fa.num_trees = forest.num_trees();
  fa.tree_off = forest.tree_off.data();
  fa.left = forest.left.data();
  fa.right = forest.right.data();
  fa.feat = forest.feat.data();
  fa.thr = forest.thr.data();
  fa.class_id = forest.num_classes > 0 ? forest.class_id.data() : nullptr;
  fa.num_classes = forest.num_classes;
  fa.transform = forest.transform;
  fa.initial_value = forest.initial_value;
  fa.num_features = opt.numberOfFeatures > 0 ? std::max(opt.numberOfFeatures, forest.num_features)
                                              : forest.num_features;
  tbk_forest *kf = nullptr;
  int rc = TBK_OK;
  if (save_image) {
    // ahead-of-time use: pack only (no device is needed) and hand the bytes back
    int smem_limit = 0;
    if (cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, g_device) != cudaSuccess) {
      cudaGetLastError();
      smem_limit = 0; // no device here: the B200 figure
    }
    tbk_image *img = nullptr;
    rc = tbk_image_create(&fa, &sched, smem_limit, &img);
    if (rc == TBK_OK) {
      uint64_t n = 0;
      rc = tbk_image_serialize(img, nullptr, 0, &n);
      if (rc == TBK_OK) {
        save_image->resize(n);
        rc = tbk_image_serialize(img, save_image->data(), n, &n);
      }
      tbk_image_free(img);
    }
    if (rc != TBK_OK) set_error(rc, tbk_last_error());
    return nullptr;
  }
  bool from_image = false;
  if (cached_image && !cached_image->empty()) {
    // a compiled-model file brought its packed image along: use it if it was packed for this
    // very layout request on a device like this one, else fall back to packing the arrays
    int smem_limit = 0;
    tbk_image *img = nullptr;
    if (cudaDeviceGetAttribute(&smem_limit, cudaDevAttrMaxSharedMemoryPerBlockOptin, g_device) == cudaSuccess &&
        tbk_image_deserialize(cached_image->data(), cached_image->size(), &img) == TBK_OK) {
      if (tbk_image_matches(img, &sched, smem_limit)) {
        rc = tbk_forest_create_from_image(img, &sched, g_device, opt.batchSize, &kf);
        from_image = rc == TBK_OK;
      }
      tbk_image_free(img);
    }
    cudaGetLastError();
  }
  if (!from_image) rc = tbk_forest_create(&fa, &sched, g_device, opt.batchSize, &kf);
  if (rc != TBK_OK) {
    set_error(rc, tbk_last_error());
    return nullptr;
  }
  auto *r = new InferenceRunner();
  r->forest = kf;
  r->batchSize = opt.batchSize;
  r->rowSize = fa.num_features;
  r->inputWidth = opt.inputElementTypeWidth;
  r->returnWidth = opt.returnTypeWidth;
  r->returnFloat = opt.returnTypeFloatType;
  r->numClasses = forest.num_classes;
  r->device = g_device;
  r->fromPackedImage = from_image;
  if (g_measure_kernel_time) tbk_set_timing(kf, 1);
  for (const int32_t dev : g_more_devices) {
    tbk_forest *extra = nullptr;
    if (tbk_forest_create(&fa, &sched, dev, opt.batchSize, &extra) != TBK_OK) {
      set_error(TBK_ERR_CUDA, tbk_last_error());
      for (tbk_forest *m : r->moreForests) tbk_forest_free(m);
      tbk_forest_free(kf);
      delete r;
      return nullptr;
    }
    r->moreForests.push_back(extra);
    r->moreDevices.push_back(dev);
  }
  return r;
}

InferenceRunner *runner_from_context(TreebeardContext *ctx) {
  if (!ctx) {
    set_error(TBK_ERR_INVALID, "null context");
    return nullptr;
  }
  if (!ctx->forestLoaded) {
    if (!load_forest(ctx->creatorType, ctx->modelPath, &ctx->forest, ctx->options.numberOfFeatures)) return nullptr;
    ctx->forestLoaded = true;
  }
  return build_runner(ctx->forest, ctx->options, ctx->hasGpuOptions ? &ctx->gpuOptions : nullptr,
                      ctx->representation);
}

// ---- compiled-model files (model_file.h) ----

tb::ModelFileOptions to_file_options(const CompilerOptions &opt, const GPUAutoScheduleOptions *gpu,
                                     const std::string &repName) {
  tb::ModelFileOptions m;
  m.batch_size = opt.batchSize;
  m.tile_size = opt.tileSize <= 0 ? 1 : opt.tileSize;
  m.threshold_width = opt.thresholdTypeWidth;
  m.feature_index_width = opt.featureIndexTypeWidth;
  m.input_width = opt.inputElementTypeWidth;
  m.return_width = opt.returnTypeWidth;
  m.return_is_float = opt.returnTypeFloatType ? 1 : 0;
  m.number_of_features = opt.numberOfFeatures > 0 ? opt.numberOfFeatures : 0;
  if (gpu) {
    m.has_gpu_options = 1;
    m.rows_per_block = gpu->numRowsPerTB;
    m.rows_per_thread = gpu->numRowsPerThread;
    m.tree_threads = gpu->numTreeThreads;
    m.cache_trees = gpu->cacheTrees ? 1 : 0;
    m.cache_rows = gpu->cacheRows ? 1 : 0;
  }
  // an unnamed representation is resolved now, so that the file does not depend on the
  // loading process's default
  m.representation = !repName.empty() ? repName : !g_rep_flag_set ? "gpu_auto" : g_use_sparse ? "gpu_sparse" : "gpu_array";
  return m;
}

void from_file_options(const tb::ModelFileOptions &m, CompilerOptions *opt, GPUAutoScheduleOptions *gpu) {
  opt->batchSize = m.batch_size;
  opt->tileSize = m.tile_size;
  opt->thresholdTypeWidth = m.threshold_width;
  opt->featureIndexTypeWidth = m.feature_index_width;
  opt->inputElementTypeWidth = m.input_width;
  opt->returnTypeWidth = m.return_width;
  opt->returnTypeFloatType = m.return_is_float != 0;
  opt->numberOfFeatures = m.number_of_features > 0 ? m.number_of_features : -1;
  gpu->numRowsPerTB = m.rows_per_block;
  gpu->numRowsPerThread = m.rows_per_thread;
  gpu->numTreeThreads = m.tree_threads;
  gpu->cacheTrees = m.cache_trees != 0;
  gpu->cacheRows = m.cache_rows != 0;
}

bool write_compiled_model(const tb::Forest &forest, const CompilerOptions &opt, const GPUAutoScheduleOptions *gpu,
                          const std::string &repName, const char *modelFilePath, const char *globalsPath) {
  if (!modelFilePath || !*modelFilePath) {
    set_error(TBK_ERR_INVALID, "no output path for the compiled-model file");
    return false;
  }
  const tb::ModelFileOptions m = to_file_options(opt, gpu, repName);
  // the packed image for the bound options travels with the forest, so that loading the file
  // skips the packer; if packing fails here the file is written without it
  std::vector<uint8_t> image;
  clear_error();
  build_runner(forest, opt, gpu, repName, nullptr, &image);
  if (g_status != TBK_OK) {
    image.clear();
    clear_error();
  }
  std::string err = tb::save_model_file(modelFilePath, forest, m, &image);
  if (err.empty() && globalsPath && *globalsPath) err = tb::save_globals_json(globalsPath, forest, m);
  if (!err.empty()) {
    set_error(TBK_ERR_IO, err);
    return false;
  }
  return true;
}

void run_batch(InferenceRunner *r, void *inputs, void *results, int64_t rows) {
  const int32_t kind = (!r->returnFloat && r->returnWidth == 8) ? TBK_OUT_I8 : TBK_OUT_F32;
  // Device buffers are an extension of the reference API (which only takes host buffers):
  // inputs and results must then lie on the same side, and device buffers on the runner's GPU.
  auto side = [](const void *ptr, int *device) {
    cudaPointerAttributes attr{};
    const bool ok = cudaPointerGetAttributes(&attr, ptr) == cudaSuccess;
    cudaGetLastError();
    *device = ok ? attr.device : -1;
    return ok && (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
  };
  int in_dev = -1, out_dev = -1;
  const bool on_device = side(inputs, &in_dev);
  const bool out_on_device = side(results, &out_dev);
  if (on_device != out_on_device) {
    set_error(TBK_ERR_INVALID, on_device ? "inputs are in device memory but results are in host memory"
                                         : "inputs are in host memory but results are in device memory");
    return;
  }
  if (on_device && (in_dev != r->device || out_dev != r->device)) {
    set_error(TBK_ERR_INVALID, "device buffers are not on the runner's GPU");
    return;
  }
  // 64-bit host buffers: convert into fp32 staging vectors around the fp32 path
  const bool wide_in = r->inputWidth == 64, wide_out = r->returnFloat && r->returnWidth == 64;
  std::vector<float> narrow_in, narrow_out;
  void *wide_results = nullptr;
  if (wide_in || wide_out) {
    if (on_device) {
      set_error(TBK_ERR_UNSUPPORTED, "64-bit inputs or results are converted on the host: pass host buffers");
      return;
    }
    if (wide_in) {
      const double *src = static_cast<const double *>(inputs);
      const int64_t n = rows * r->rowSize;
      narrow_in.resize((size_t)n);
#pragma omp parallel for schedule(static)
      for (int64_t i = 0; i < n; ++i) narrow_in[i] = (float)src[i];
      inputs = narrow_in.data();
    }
    if (wide_out) {
      narrow_out.resize((size_t)rows);
      wide_results = results;
      results = narrow_out.data();
    }
  }
  int rc = TBK_OK;
  const int runs = g_measure_kernel_time ? std::max(1, g_kernel_runs) : 1;
  if (on_device) {
    for (int i = 0; i < runs && rc == TBK_OK; ++i) {
      rc = tbk_predict(r->forest, static_cast<const float *>(inputs), rows, r->rowSize, results, kind, nullptr);
      if (rc == TBK_OK && g_measure_kernel_time) {
        const int64_t us = tbk_last_kernel_time_us(r->forest);
        if (us > 0) r->kernelMicros += us;
      }
    }
    if (rc == TBK_OK && cudaDeviceSynchronize() != cudaSuccess) {
      rc = TBK_ERR_CUDA;
      set_error(rc, "cudaDeviceSynchronize failed after the walk");
      return;
    }
    if (rc == TBK_OK) rc = tbk_check_status(r->forest);
  } else if (g_measure_kernel_time) {
    // timed mode: copy once, then time the kernel alone, as the reference's
    // generated host code does around its launch
    float *d_in = nullptr;
    void *d_out = nullptr;
    const size_t in_bytes = (size_t)rows * r->rowSize * 4, out_bytes = (size_t)rows * (kind == TBK_OUT_I8 ? 1 : 4);
    if (cudaMalloc(reinterpret_cast<void **>(&d_in), in_bytes) != cudaSuccess || cudaMalloc(&d_out, out_bytes) != cudaSuccess ||
        cudaMemcpy(d_in, inputs, in_bytes, cudaMemcpyHostToDevice) != cudaSuccess) {
      cudaFree(d_in);
      cudaFree(d_out);
      set_error(TBK_ERR_CUDA, "device staging for the timed run failed");
      return;
    }
    for (int i = 0; i < runs && rc == TBK_OK; ++i) {
      rc = tbk_predict(r->forest, d_in, rows, r->rowSize, d_out, kind, nullptr);
      if (rc == TBK_OK) {
        const int64_t us = tbk_last_kernel_time_us(r->forest);
        if (us > 0) r->kernelMicros += us;
      }
    }
    if (rc == TBK_OK && cudaMemcpy(results, d_out, out_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) rc = TBK_ERR_CUDA;
    cudaFree(d_in);
    cudaFree(d_out);
    if (rc == TBK_OK) rc = tbk_check_status(r->forest);
  } else if (!r->moreForests.empty() && rows >= 64 * (int64_t)(1 + r->moreForests.size())) {
    // one contiguous row range per device (multiples of 32 rows), predicted concurrently
    const int64_t parts = 1 + (int64_t)r->moreForests.size();
    const int64_t share = ((rows + parts - 1) / parts + 31) / 32 * 32;
    const size_t out_elt = kind == TBK_OUT_I8 ? 1 : 4;
    std::vector<int> codes((size_t)parts, TBK_OK);
    std::vector<std::string> messages((size_t)parts);
    std::vector<std::thread> workers;
    for (int64_t k = 0; k < parts; ++k) {
      const int64_t lo = std::min(rows, k * share), n = std::min(rows, lo + share) - lo;
      if (n <= 0) continue;
      tbk_forest *forest = k == 0 ? r->forest : r->moreForests[(size_t)k - 1];
      workers.emplace_back([=, &codes, &messages] {
        codes[(size_t)k] = tbk_predict_host(forest, static_cast<const float *>(inputs) + lo * r->rowSize, n, r->rowSize,
                                            static_cast<unsigned char *>(results) + (size_t)lo * out_elt, kind);
        if (codes[(size_t)k] != TBK_OK) messages[(size_t)k] = tbk_last_error(); // (the message is per thread)
      });
    }
    for (std::thread &w : workers) w.join();
    for (int64_t k = 0; k < parts; ++k)
      if (codes[(size_t)k] != TBK_OK) {
        set_error(codes[(size_t)k], messages[(size_t)k]);
        return;
      }
  } else {
    rc = tbk_predict_host(r->forest, static_cast<const float *>(inputs), rows, r->rowSize, results, kind);
  }
  if (rc != TBK_OK) {
    set_error(rc, tbk_last_error());
    return;
  }
  if (wide_results) {
    double *dst = static_cast<double *>(wide_results);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < rows; ++i) dst[i] = (double)narrow_out[i];
  }
}

} // namespace

extern "C" {

int32_t TB_GetLastStatus(void) { return g_status; }
const char *TB_GetLastError(void) { return g_error.c_str(); }
void TB_SetDevice(int32_t device) {
  g_device = device;
  g_more_devices.clear();
}
void TB_SetDevices(const int32_t *devices, int32_t count) {
  if (!devices || count <= 0) return;
  g_device = devices[0];
  g_more_devices.assign(devices + 1, devices + count);
}
int32_t TB_RunnerDeviceCount(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r ? 1 + (int32_t)r->moreForests.size() : 0;
}

// ---- execution ----

intptr_t InitializeInferenceRunner(const char *modelFilePath, const char *modelGlobalsJSONPath) {
  clear_error();
  if (!modelFilePath) {
    set_error(TBK_ERR_INVALID, "null argument");
    return 0;
  }
  tb::Forest forest;
  tb::ModelFileOptions m;
  std::vector<uint8_t> image;
  std::string err = tb::load_model_file(modelFilePath, &forest, &m, &image);
  if (err.empty() && modelGlobalsJSONPath && *modelGlobalsJSONPath) err = tb::load_globals_json(modelGlobalsJSONPath, &m);
  if (!err.empty()) {
    set_error(TBK_ERR_IO, err);
    return 0;
  }
  CompilerOptions opt;
  GPUAutoScheduleOptions gpu;
  from_file_options(m, &opt, &gpu);
  return reinterpret_cast<intptr_t>(build_runner(forest, opt, m.has_gpu_options ? &gpu : nullptr, m.representation, &image));
}

void RunInference(intptr_t runner, void *inputs, void *results) {
  clear_error();
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  if (!r || !inputs || !results) return set_error(TBK_ERR_INVALID, "null argument");
  run_batch(r, inputs, results, r->batchSize);
}

void RunInferenceOnMultipleBatches(intptr_t runner, void *inputs, void *results, int32_t numRows) {
  clear_error();
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  if (!r || !inputs || !results) return set_error(TBK_ERR_INVALID, "null argument");
  if (numRows < 0 || numRows % r->batchSize != 0)
    return set_error(TBK_ERR_INVALID, "the number of rows must be a multiple of the batch size");
  // batches are independent and contiguous: one pipelined pass covers them all
  run_batch(r, inputs, results, numRows);
}

int32_t GetBatchSize(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r ? r->batchSize : 0;
}
int32_t GetRowSize(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r ? r->rowSize : 0;
}
int32_t TB_GetInputTypeBitWidth(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r ? r->inputWidth : 0;
}
int32_t TB_GetReturnTypeBitWidth(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r ? r->returnWidth : 0;
}
void DeleteInferenceRunner(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  if (!r) return;
  tbk_forest_free(r->forest);
  for (tbk_forest *m : r->moreForests) tbk_forest_free(m);
  delete r;
}
int32_t TB_RunnerUsedPackedImage(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r && r->fromPackedImage ? 1 : 0;
}
void *TB_GetKernelForest(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return r ? r->forest : nullptr;
}
int64_t GetGPUKernelExecutionTime(intptr_t runner) {
  auto *r = reinterpret_cast<InferenceRunner *>(runner);
  return (r && g_measure_kernel_time) ? r->kernelMicros : 0;
}

// ---- compiler options ----

intptr_t CreateCompilerOptions(void) { return reinterpret_cast<intptr_t>(new CompilerOptions()); }
void DeleteCompilerOptions(intptr_t o) { delete reinterpret_cast<CompilerOptions *>(o); }

#define OPTION_SETTER(name, type, expr)                                      \
  void Set_##name(intptr_t o, type val) {                                    \
    auto *opt = reinterpret_cast<CompilerOptions *>(o);                      \
    if (opt) opt->name = (expr);                                             \
  }
OPTION_SETTER(numberOfFeatures, int32_t, val)
OPTION_SETTER(batchSize, int32_t, val)
OPTION_SETTER(tileSize, int32_t, val)
OPTION_SETTER(thresholdTypeWidth, int32_t, val)
OPTION_SETTER(returnTypeWidth, int32_t, val)
OPTION_SETTER(returnTypeFloatType, int32_t, val != 0)
OPTION_SETTER(featureIndexTypeWidth, int32_t, val)
OPTION_SETTER(nodeIndexTypeWidth, int32_t, val)
OPTION_SETTER(inputElementTypeWidth, int32_t, val)
OPTION_SETTER(tileShapeBitWidth, int32_t, val)
OPTION_SETTER(childIndexBitWidth, int32_t, val)
OPTION_SETTER(makeAllLeavesSameDepth, int32_t, val != 0)
OPTION_SETTER(reorderTreesByDepth, int32_t, val != 0)
OPTION_SETTER(statsProfileCSVPath, const char *, std::string(val ? val : ""))
OPTION_SETTER(pipelineSize, int32_t, val)
OPTION_SETTER(numberOfCores, int32_t, val)
OPTION_SETTER(numParallelTreeBatches, int32_t, val)
OPTION_SETTER(tilingType, int32_t, val)
#undef OPTION_SETTER

void SetOneTreeAtATimeSchedule(intptr_t o) {
  auto *opt = reinterpret_cast<CompilerOptions *>(o);
  if (opt) opt->oneTreeAtATime = true; // the kernels already walk one tree group at a time
}

// ---- GPU auto-schedule options ----

intptr_t CreateGPUAutoScheduleOptions(void) { return reinterpret_cast<intptr_t>(new GPUAutoScheduleOptions()); }
void DeleteGPUAutoScheduleOptions(intptr_t o) { delete reinterpret_cast<GPUAutoScheduleOptions *>(o); }
#define GPU_OPTION_SETTER(name, expr)                                        \
  void Set_##name(intptr_t o, int32_t val) {                                 \
    auto *opt = reinterpret_cast<GPUAutoScheduleOptions *>(o);               \
    if (opt) opt->name = (expr);                                             \
  }
GPU_OPTION_SETTER(numRowsPerTB, val)
GPU_OPTION_SETTER(numRowsPerThread, val)
GPU_OPTION_SETTER(rowTileSize, val)
GPU_OPTION_SETTER(numTreeThreads, val)
GPU_OPTION_SETTER(numTreesAtATime, val)
GPU_OPTION_SETTER(cacheRows, val != 0)
GPU_OPTION_SETTER(cacheTrees, val != 0)
GPU_OPTION_SETTER(unrollTreeWalks, val != 0)
GPU_OPTION_SETTER(treeWalkInterleaveFactor, val)
GPU_OPTION_SETTER(sharedMemoryReduce, val != 0)
#undef GPU_OPTION_SETTER

// ---- one-call construction ----

// The reference's ahead-of-time flow writes LLVM IR (compiled to a shared object by the
// user) plus a globals JSON, and InitializeInferenceRunner loads the pair back.  There is
// no LLVM back end here: the same two calls write the compiled-model file (binary forest +
// bound options) to the second path and the globals JSON to the third, and
// InitializeInferenceRunner loads that pair.
void GenerateLLVMIRForXGBoostModel(const char *modelJSONPath, const char *modelFilePath, const char *globalsPath,
                                   intptr_t options) {
  clear_error();
  auto *opt = reinterpret_cast<CompilerOptions *>(options);
  if (!modelJSONPath || !opt) return set_error(TBK_ERR_INVALID, "null argument");
  tb::Forest forest;
  if (!load_forest("xgboost_json", modelJSONPath, &forest)) return;
  write_compiled_model(forest, *opt, nullptr, "", modelFilePath, globalsPath);
}
void CreateLLVMIRForONNXModel(const char *modelPath, const char *modelFilePath, const char *globalsPath,
                              intptr_t options) {
  clear_error();
  auto *opt = reinterpret_cast<CompilerOptions *>(options);
  if (!modelPath || !opt) return set_error(TBK_ERR_INVALID, "null argument");
  tb::Forest forest;
  if (!load_forest("onnx_file", modelPath, &forest, opt->numberOfFeatures)) return;
  write_compiled_model(forest, *opt, nullptr, "", modelFilePath, globalsPath);
}

intptr_t CreateInferenceRunner(const char *modelJSONPath, const char *, intptr_t options) {
  clear_error();
  auto *opt = reinterpret_cast<CompilerOptions *>(options);
  if (!modelJSONPath || !opt) {
    set_error(TBK_ERR_INVALID, "null argument");
    return 0;
  }
  tb::Forest forest;
  if (!load_forest("xgboost_json", modelJSONPath, &forest)) return 0;
  return reinterpret_cast<intptr_t>(build_runner(forest, *opt, nullptr, ""));
}

intptr_t CreateInferenceRunnerForONNXModel(const char *modelPath, intptr_t options) {
  clear_error();
  auto *opt = reinterpret_cast<CompilerOptions *>(options);
  if (!modelPath || !opt) {
    set_error(TBK_ERR_INVALID, "null argument");
    return 0;
  }
  tb::Forest forest;
  if (!load_forest("onnx_file", modelPath, &forest, opt->numberOfFeatures)) return 0;
  return reinterpret_cast<intptr_t>(build_runner(forest, *opt, nullptr, ""));
}

intptr_t TB_CreateInferenceRunnerFromArrays(const void *forestArrays, intptr_t options, intptr_t gpuOptions,
                                            const char *representation) {
  clear_error();
  auto *fa = static_cast<const tbk_forest_arrays *>(forestArrays);
  auto *opt = reinterpret_cast<CompilerOptions *>(options);
  if (!fa || !opt || fa->num_trees <= 0) {
    set_error(TBK_ERR_INVALID, "null or empty argument");
    return 0;
  }
  tb::Forest f;
  const int64_t T = fa->num_trees, N = fa->tree_off[T];
  f.tree_off.assign(fa->tree_off, fa->tree_off + T + 1);
  f.left.assign(fa->left, fa->left + N);
  f.right.assign(fa->right, fa->right + N);
  f.feat.assign(fa->feat, fa->feat + N);
  f.thr.assign(fa->thr, fa->thr + N);
  if (fa->class_id) f.class_id.assign(fa->class_id, fa->class_id + T);
  else f.class_id.assign(T, 0);
  f.num_classes = fa->num_classes;
  f.transform = fa->transform;
  f.initial_value = fa->initial_value;
  f.num_features = fa->num_features;
  return reinterpret_cast<intptr_t>(build_runner(f, *opt, reinterpret_cast<GPUAutoScheduleOptions *>(gpuOptions),
                                                 representation ? representation : ""));
}

// ---- host-side model loading (no device involved) ----

intptr_t TB_LoadForest(const char *modelPath, const char *creatorType, int32_t numberOfFeatures) {
  clear_error();
  if (!modelPath || !creatorType) {
    set_error(TBK_ERR_INVALID, "null argument");
    return 0;
  }
  auto *f = new tb::Forest();
  if (!load_forest(creatorType, modelPath, f, numberOfFeatures)) {
    delete f;
    return 0;
  }
  return reinterpret_cast<intptr_t>(f);
}

int32_t TB_ForestGetArrays(intptr_t forest, void *arraysOut) {
  auto *f = reinterpret_cast<tb::Forest *>(forest);
  auto *fa = static_cast<tbk_forest_arrays *>(arraysOut);
  if (!f || !fa) return TBK_ERR_INVALID;
  fa->num_trees = f->num_trees();
  fa->tree_off = f->tree_off.data();
  fa->left = f->left.data();
  fa->right = f->right.data();
  fa->feat = f->feat.data();
  fa->thr = f->thr.data();
  fa->class_id = f->class_id.data();
  fa->num_classes = f->num_classes;
  fa->transform = f->transform;
  fa->initial_value = f->initial_value;
  fa->num_features = f->num_features;
  return TBK_OK;
}

void TB_FreeForest(intptr_t forest) { delete reinterpret_cast<tb::Forest *>(forest); }

// ---- process-wide switches ----

void SetEnableSparseRepresentation(int32_t val) {
  g_use_sparse = val != 0;
  g_rep_flag_set = true;
}
int32_t IsSparseRepresentationEnabled(void) { return g_use_sparse; }
void SetPeeledCodeGenForProbabilityBasedTiling(int32_t val) { g_peeled_codegen = val != 0; }
int32_t IsPeeledCodeGenForProbabilityBasedTilingEnabled(void) { return g_peeled_codegen; }
void SetEnableMeasureGpuKernelTime(bool val) { g_measure_kernel_time = val; }
void SetNumberOfKernelRuns(int32_t val) { g_kernel_runs = val; }

// ---- representation objects ----

void *ConstructRepresentation(const char *repName) {
  clear_error();
  if (!repName || rep_from_name(repName) < TBK_REP_AUTO) {
    set_error(TBK_ERR_INVALID, "unknown representation");
    return nullptr;
  }
  auto *s = new std::string(repName);
  std::lock_guard<std::mutex> lock(g_live_mu);
  g_representations.insert(s);
  return s;
}
void DestroyRepresentation(void *rep) {
  std::lock_guard<std::mutex> lock(g_live_mu);
  if (g_representations.erase(rep)) delete static_cast<std::string *>(rep);
}

// ---- context ----

intptr_t ConstructTreebeardContext(const char *modelPath, const char *globalsPath, intptr_t options) {
  clear_error();
  auto *opt = reinterpret_cast<CompilerOptions *>(options);
  if (!modelPath || !opt) {
    set_error(TBK_ERR_INVALID, "null argument");
    return 0;
  }
  auto *ctx = new TreebeardContext();
  ctx->modelPath = modelPath;
  ctx->globalsPath = globalsPath ? globalsPath : "";
  ctx->options = *opt;
  return reinterpret_cast<intptr_t>(ctx);
}

intptr_t ConstructTreebeardContextFromGPUAutoscheduleOptions(const char *modelPath, const char *globalsPath,
                                                             intptr_t options, intptr_t gpuOptions) {
  intptr_t h = ConstructTreebeardContext(modelPath, globalsPath, options);
  auto *ctx = reinterpret_cast<TreebeardContext *>(h);
  auto *gpu = reinterpret_cast<GPUAutoScheduleOptions *>(gpuOptions);
  if (ctx && gpu) {
    ctx->gpuOptions = *gpu;
    ctx->hasGpuOptions = true;
    // unrolled walks need every leaf at the same depth (src/runtime/runtime.cpp:784-785);
    // the kernels always walk a fixed depth, so this only records the request
    if (gpu->unrollTreeWalks) ctx->options.makeAllLeavesSameDepth = true;
  }
  return h;
}

void DestroyTreebeardContext(intptr_t c) { delete reinterpret_cast<TreebeardContext *>(c); }

void SetForestCreatorType(intptr_t c, const char *creatorType) {
  clear_error();
  auto *ctx = reinterpret_cast<TreebeardContext *>(c);
  if (!ctx || !creatorType) return set_error(TBK_ERR_INVALID, "null argument");
  const std::string name = creatorType;
  if (name != "xgboost_json" && name != "onnx_file")
    return set_error(TBK_ERR_INVALID, "unknown forest creator \"" + name + "\"");
  ctx->creatorType = name;
  ctx->forestLoaded = false;
}

void SetRepresentationAndSerializer(intptr_t c, const char *repType) {
  clear_error();
  auto *ctx = reinterpret_cast<TreebeardContext *>(c);
  if (!ctx || !repType) return set_error(TBK_ERR_INVALID, "null argument");
  if (rep_from_name(repType) < TBK_REP_AUTO) return set_error(TBK_ERR_INVALID, std::string("unknown representation \"") + repType + "\"");
  ctx->representation = repType;
}

void BuildHIRRepresentation(void *c) {
  clear_error();
  auto *ctx = static_cast<TreebeardContext *>(c);
  if (!ctx) return set_error(TBK_ERR_INVALID, "null context");
  if (!ctx->forestLoaded) {
    if (!load_forest(ctx->creatorType, ctx->modelPath, &ctx->forest, ctx->options.numberOfFeatures)) return;
    ctx->forestLoaded = true;
  }
  if (!ctx->schedule)
    ctx->schedule.reset(new Schedule(ctx->options.batchSize, (int32_t)ctx->forest.num_trees()));
}

void *GetScheduleFromTBContext(intptr_t c) {
  auto *ctx = reinterpret_cast<TreebeardContext *>(c);
  if (!ctx) return nullptr;
  if (!ctx->schedule) BuildHIRRepresentation(ctx);
  return ctx->schedule.get();
}

// Writes the context's compiled-model file to fileName and, when the context was given a
// globals path, the globals JSON there (the reference dumps LLVM IR and its serializer's
// globals file at this point: src/runtime/runtime.cpp:434-440).
bool LowerToLLVMAndDumpIR(void *c, const char *fileName) {
  clear_error();
  auto *ctx = static_cast<TreebeardContext *>(c);
  if (!ctx) {
    set_error(TBK_ERR_INVALID, "null context");
    return false;
  }
  if (!ctx->forestLoaded) {
    if (!load_forest(ctx->creatorType, ctx->modelPath, &ctx->forest, ctx->options.numberOfFeatures)) return false;
    ctx->forestLoaded = true;
  }
  return write_compiled_model(ctx->forest, ctx->options, ctx->hasGpuOptions ? &ctx->gpuOptions : nullptr,
                              ctx->representation, fileName, ctx->globalsPath.c_str());
}

void *ConstructInferenceRunnerFromHIR(void *c) {
  clear_error();
  return runner_from_context(static_cast<TreebeardContext *>(c));
}
void *ConstructGPUInferenceRunnerFromHIR(void *c) {
  clear_error();
  return runner_from_context(static_cast<TreebeardContext *>(c));
}
void *ConstructGPUInferenceRunnerFromTBContext(void *c) {
  clear_error();
  return runner_from_context(static_cast<TreebeardContext *>(c));
}
void *findBestGPUScheduleAndCompileModel(void *c) {
  clear_error();
  auto *ctx = static_cast<TreebeardContext *>(c);
  if (!ctx) {
    set_error(TBK_ERR_INVALID, "null context");
    return nullptr;
  }
  // the selector replaces the timed search over schedules and representations: drop any
  // pinned launch shape and let the library choose the layout for this forest as well
  ctx->hasGpuOptions = false;
  ctx->representation = "gpu_auto";
  return runner_from_context(ctx);
}

// ---- schedule objects ----

#define SCHED(p) reinterpret_cast<Schedule *>(p)
#define IDX(p) reinterpret_cast<IndexVariable *>(p)

intptr_t Schedule_NewIndexVariable(intptr_t s, const char *name) {
  return s ? reinterpret_cast<intptr_t>(SCHED(s)->add(name ? name : "")) : 0;
}
intptr_t Schedule_NewIndexVariable2(intptr_t s, intptr_t v) {
  return (s && v) ? reinterpret_cast<intptr_t>(SCHED(s)->add(IDX(v)->name)) : 0;
}
void Schedule_Tile(intptr_t s, intptr_t i, intptr_t o, intptr_t in, int32_t tileSize) {
  if (!s) return;
  std::ostringstream os;
  os << "tile(" << name_of(IDX(i)) << " -> " << name_of(IDX(o)) << ", " << name_of(IDX(in)) << ", " << tileSize << ")";
  SCHED(s)->note(os.str());
}
void Schedule_Reorder(intptr_t s, intptr_t indices, int32_t n) {
  if (!s) return;
  std::ostringstream os;
  os << "reorder(";
  auto **arr = reinterpret_cast<IndexVariable **>(indices);
  for (int32_t k = 0; arr && k < n; ++k) os << (k ? ", " : "") << name_of(arr[k]);
  os << ")";
  SCHED(s)->note(os.str());
}
void Schedule_Split(intptr_t s, intptr_t i, intptr_t a, intptr_t b, int32_t at, intptr_t) {
  if (!s) return;
  std::ostringstream os;
  os << "split(" << name_of(IDX(i)) << " -> " << name_of(IDX(a)) << ", " << name_of(IDX(b)) << " at " << at << ")";
  SCHED(s)->note(os.str());
}
intptr_t Schedule_Specialize(intptr_t s, intptr_t i) {
  if (s) SCHED(s)->note(std::string("specialize(") + name_of(IDX(i)) + ")");
  return 0;
}
int64_t GetSpecializationInfoNumIterations(intptr_t) { return 0; }
int64_t GetSpecializationInfoNumEntries(intptr_t) { return 0; }
void GetSpecializationInfoEntries(intptr_t, intptr_t, intptr_t) {}
void Schedule_Pipeline(intptr_t s, intptr_t i, int32_t step) {
  if (s) SCHED(s)->note(std::string("pipeline(") + name_of(IDX(i)) + ", " + std::to_string(step) + ")");
}
void Schedule_Simdize(intptr_t s, intptr_t i) { if (s) SCHED(s)->note(std::string("simdize(") + name_of(IDX(i)) + ")"); }
void Schedule_Parallel(intptr_t s, intptr_t i) { if (s) SCHED(s)->note(std::string("parallel(") + name_of(IDX(i)) + ")"); }
void Schedule_Unroll(intptr_t s, intptr_t i) { if (s) SCHED(s)->note(std::string("unroll(") + name_of(IDX(i)) + ")"); }
void Schedule_PeelWalk(intptr_t s, intptr_t i, int32_t n) {
  if (s) SCHED(s)->note(std::string("peelWalk(") + name_of(IDX(i)) + ", " + std::to_string(n) + ")");
}
void Schedule_Cache(intptr_t s, intptr_t i) { if (s) SCHED(s)->note(std::string("cache(") + name_of(IDX(i)) + ")"); }
intptr_t Schedule_GetRootIndex(intptr_t s) { return s ? reinterpret_cast<intptr_t>(SCHED(s)->batch) : 0; }
intptr_t Schedule_GetBatchIndex(intptr_t s) { return s ? reinterpret_cast<intptr_t>(SCHED(s)->batch) : 0; }
intptr_t Schedule_GetTreeIndex(intptr_t s) { return s ? reinterpret_cast<intptr_t>(SCHED(s)->tree) : 0; }
int32_t Schedule_PrintToString(intptr_t s, intptr_t str, int32_t len) {
  if (!s) return -1;
  std::ostringstream os;
  os << "for batch in [0, " << SCHED(s)->batchSize << ") x tree in [0, " << SCHED(s)->forestSize << ")";
  for (auto &d : SCHED(s)->directives) os << "; " << d;
  const std::string text = os.str();
  // as the reference: -1 when the buffer is too small, else the text length
  if (!str || len < (int32_t)text.size() + 1) return -1;
  std::memcpy(reinterpret_cast<char *>(str), text.c_str(), text.size() + 1);
  return (int32_t)text.size();
}
int32_t Schedule_GetBatchSize(intptr_t s) { return s ? SCHED(s)->batchSize : 0; }
int32_t Schedule_GetForestSize(intptr_t s) { return s ? SCHED(s)->forestSize : 0; }
bool Schedule_IsDefaultSchedule(intptr_t s) { return s ? !SCHED(s)->touched : true; }
void Schedule_Finalize(intptr_t) {}
void Schedule_AtomicReduce(intptr_t s, intptr_t i) { if (s) SCHED(s)->note(std::string("atomicReduce(") + name_of(IDX(i)) + ")"); }
void Schedule_VectorReduce(intptr_t s, intptr_t i, int32_t w) {
  if (s) SCHED(s)->note(std::string("vectorReduce(") + name_of(IDX(i)) + ", " + std::to_string(w) + ")");
}
void Schedule_SharedReduce(intptr_t s, intptr_t i) { if (s) SCHED(s)->note(std::string("sharedReduce(") + name_of(IDX(i)) + ")"); }
void IndexVariable_SetGPUThreadDim(intptr_t v, int32_t construct, int32_t dim) {
  if (!v) return;
  IDX(v)->gpuConstruct = construct;
  IDX(v)->gpuDim = dim;
}
#undef SCHED
#undef IDX

} // extern "C"
