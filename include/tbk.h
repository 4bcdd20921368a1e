/*
 * tbk.h -- C ABI of the B200 tree-ensemble inference kernels.
 *
 * This is the inner boundary of the library: the place where, in the reference,
 * the inference runner calls into the generated module (Init_* uploads,
 * Prediction_Function, Dealloc_Buffers -- resolved by name in
 * src/mlir/ExecutionHelpers.cpp:37-51 and src/gpu/GPUModelSerializers.cpp:21-262).
 * Every entry point takes plain pointers and sizes, returns an int status
 * (0 = success) and never aborts; the message of the last failure on the calling
 * thread is available from tbk_last_error().
 *
 * Device pointers are raw CUDA device addresses; `stream` is a cudaStream_t passed
 * as void* (NULL = the legacy default stream).
 */
#ifndef TBK_H
#define TBK_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TBK_EXPORT __attribute__((visibility("default")))

/* status codes */
enum {
  TBK_OK = 0,
  TBK_ERR_INVALID = 1,     /* bad argument / malformed forest */
  TBK_ERR_CUDA = 2,        /* a CUDA runtime call failed */
  TBK_ERR_UNSUPPORTED = 3, /* valid request outside what the kernels cover */
  TBK_ERR_DEVICE_WAIT = 4, /* a bounded device-side wait expired */
  TBK_ERR_IO = 5           /* file could not be read / parsed */
};

/* prediction transformations (src/include/DecisionForest.h:26) */
enum { TBK_IDENTITY = 0, TBK_SIGMOID = 1, TBK_SOFTMAX = 2 };

/* packed-forest representations
 * (factory names in src/mlir/Representations.h:364-380 and
 *  src/gpu/GPURepresentations.cpp:1238,1982, src/gpu/ReorgForestRepresentation.cpp:390) */
enum { TBK_REP_AUTO = -1, TBK_REP_SPARSE = 0, TBK_REP_ARRAY = 1, TBK_REP_REORG = 2 };

/* output element kinds: fp32 prediction, or int8 class id for a multiclass forest
 * (the reference's multiclass return type, test/python/gpu_tests.py:133-136) */
enum { TBK_OUT_F32 = 0, TBK_OUT_I8 = 1 };

/*
 * Host-side forest as flat arrays: tree t owns nodes [tree_off[t], tree_off[t+1]);
 * left/right are node indices inside the tree, -1/-1 marks a leaf; thr is the split
 * threshold or, for a leaf, the leaf value (the reference keeps leaf values in the
 * threshold field too: src/include/DecisionForest.h:35-54).  Replaces the in-memory
 * model the reference's front end builds (src/json/xgboostparser.h:116-219).
 */
typedef struct tbk_forest_arrays {
  int64_t num_trees;
  const int64_t *tree_off;
  const int32_t *left;
  const int32_t *right;
  const int32_t *feat;
  const float *thr;
  const int32_t *class_id; /* per tree; may be NULL when num_classes == 0 */
  int32_t num_classes;     /* 0 = single output */
  int32_t transform;       /* TBK_IDENTITY / TBK_SIGMOID / TBK_SOFTMAX */
  double initial_value;
  int32_t num_features;
} tbk_forest_arrays;

/*
 * Schedule: the knobs of the reference's GPU auto-schedule options
 * (src/include/TreebeardContext.h:138-162) mapped onto the fixed kernel family.
 * A zero in any field means "let the selector choose".
 */
typedef struct tbk_schedule {
  int32_t representation;  /* TBK_REP_*; TBK_REP_AUTO lets the selector choose */
  int32_t tile_size;       /* nodes per tile, 1..4 (0 = 1) */
  int32_t rows_per_block;  /* numRowsPerTB */
  int32_t rows_per_thread; /* numRowsPerThread: rows walked in lock-step by a lane */
  int32_t tree_threads;    /* numTreeThreads: warps sharing a row tile, each on
                              its own subset of trees */
  int32_t tree_chunks;     /* grid.y: independent tree ranges whose partial sums are
                              combined by an atomic-free second pass */
  int32_t cache_trees;     /* 1 = stage tree groups in shared memory with bulk
                              async copies, 2 = read nodes from global memory,
                              0 = auto */
  int32_t feature_bits;    /* how rows are staged in shared memory: 32 = fp32 values,
                              16 = order-preserving 15/16-bit keys with exact fp32 tie
                              resolution (leaf selection stays bit-exact): single-output
                              forests of at most 12 levels; multiclass forests of at most
                              8 levels over narrow rows (walked in one tree chunk),
                              0 = auto: with representation TBK_REP_AUTO keys for these
                              forests unless most thresholds are whole numbers that cannot
                              become lattice features (integer-valued features then tie
                              all the time), fp32 otherwise */
  int32_t reserved[4];
} tbk_schedule;

typedef struct tbk_forest tbk_forest; /* opaque: packed forest resident on a device */

typedef struct tbk_forest_info {
  int64_t num_trees, num_nodes, num_groups;
  int64_t packed_bytes;      /* bytes of node tiles resident on the device */
  int32_t max_depth;         /* decision levels on the deepest root-to-leaf path */
  int32_t num_features, num_classes, transform;
  int32_t device;
  tbk_schedule schedule;     /* the schedule the selector settled on */
  int32_t staged;            /* 1 if tree groups are staged through shared memory */
  int32_t smem_bytes;        /* dynamic shared memory per block of the walk kernel */
  int32_t threads_per_block;
  int32_t reserved[8];
} tbk_forest_info;

/* Packs the forest in the requested representation and uploads it to `device`.
 * Replaces Init_Model / Init_Offsets / Init_Lengths / Init_ClassIds / Init_LUT /
 * Init_Thresholds / Init_FeatureIndices (src/gpu/GPURepresentations.cpp:22-256,
 * src/gpu/ReorgForestRepresentation.cpp:400-487) and the host-side lowering that
 * feeds them (src/utils/TreeTilingUtils.cpp:427-556).  `schedule` may be NULL. */
TBK_EXPORT int tbk_forest_create(const tbk_forest_arrays *forest, const tbk_schedule *schedule,
                                 int32_t device, int64_t batch_hint, tbk_forest **out);

/* The two halves of tbk_forest_create.  An image is the packed forest in host memory: the
 * layout chosen for it and that layout's buffers (what the reference's serializers build with
 * the host-side lowering of src/utils/TreeTilingUtils.cpp:427-556 before Init_* uploads them).
 * tbk_image_create needs no device: smem_limit is the shared memory per block the layout is
 * chosen for (0 = 227 KB, the B200 figure).  An image can be turned into bytes and back, which
 * is what a compiled-model file caches (the reference reloads its serialized buffers the same
 * way: src/utils/TreeTilingUtils.cpp:95-170, src/runtime/runtime.cpp:35-54); stale or damaged
 * bytes are refused with TBK_ERR_IO.  tbk_image_matches tells whether an image was packed for
 * the same layout request (representation, tile size, feature bits of `schedule`; shared-memory
 * limit) and may therefore stand in for a fresh pack.  tbk_forest_create_from_image uploads it;
 * of `schedule` it takes the launch-shape fields, the layout is the image's. */
typedef struct tbk_image tbk_image;
TBK_EXPORT int tbk_image_create(const tbk_forest_arrays *forest, const tbk_schedule *schedule,
                                int32_t smem_limit, tbk_image **out);
TBK_EXPORT int tbk_image_free(tbk_image *image);
/* buffer == NULL: only *size is set */
TBK_EXPORT int tbk_image_serialize(const tbk_image *image, void *buffer, uint64_t capacity, uint64_t *size);
TBK_EXPORT int tbk_image_deserialize(const void *buffer, uint64_t size, tbk_image **out);
TBK_EXPORT int tbk_image_matches(const tbk_image *image, const tbk_schedule *schedule, int32_t smem_limit);
TBK_EXPORT int tbk_forest_create_from_image(const tbk_image *image, const tbk_schedule *schedule,
                                            int32_t device, int64_t batch_hint, tbk_forest **out);

/* Frees the device buffers (Dealloc_Buffers, src/gpu/GPUModelSerializers.cpp:231-262). */
TBK_EXPORT int tbk_forest_free(tbk_forest *forest);

TBK_EXPORT int tbk_forest_get_info(const tbk_forest *forest, tbk_forest_info *info);

/* Replaces the kernel inside Prediction_Function (loop nest built by
 * src/mlir/GPUAutoSchedule.cpp:318-472; walk src/mlir/CodeGenStateMachine.cpp:149-243;
 * reduction src/reduction/LowerReduceOps.cpp:921-1003; initial value and sigmoid
 * src/mlir/LowerToMidLevelIR.cpp:596-648; class argmax
 * src/reduction/LowerReduceOps.cpp:148-189).  Rows are row-major with `ld` floats
 * between rows; inputs and outputs are device-resident; stream-ordered.
 * out_kind TBK_OUT_F32: n_rows floats (class id as a float for multiclass);
 * TBK_OUT_I8: n_rows int8 class ids (multiclass only). */
TBK_EXPORT int tbk_predict(tbk_forest *forest, const float *d_rows, int64_t n_rows, int64_t ld,
                           void *d_out, int32_t out_kind, void *stream);

/* Raw per-row sums of leaf values (n_rows x max(1, num_classes) floats, row-major):
 * no initial value, no transformation.  This is what a tree shard contributes before
 * the cross-device sum; tbk_finalize() turns summed partials into predictions. */
TBK_EXPORT int tbk_predict_partial(tbk_forest *forest, const float *d_rows, int64_t n_rows,
                                   int64_t ld, float *d_partial, void *stream);
TBK_EXPORT int tbk_finalize(tbk_forest *forest, const float *d_partial, int64_t n_rows,
                            void *d_out, int32_t out_kind, void *stream);

/* Selected leaf per (row, tree): n_rows x num_trees int32, the leaf's node index in
 * the numbering of the tbk_forest_arrays the forest was created from (the quantity
 * the reference's tests observe through DecisionTree::PredictTree,
 * src/include/DecisionForest.h:347-379). */
TBK_EXPORT int tbk_predict_leaf_ids(tbk_forest *forest, const float *d_rows, int64_t n_rows,
                                    int64_t ld, int32_t *d_leaf_ids, void *stream);

/* Host-buffer variant of tbk_predict: the per-call H2D copy of the batch, the kernel
 * and the D2H copy of the results that the reference's generated host code performs
 * around its launch (src/gpu/GPUSupportUtils.cpp:150-343), here chunked and
 * overlapped on two streams.  Blocks until the results are in h_out. */
TBK_EXPORT int tbk_predict_host(tbk_forest *forest, const float *h_rows, int64_t n_rows,
                                int64_t ld, void *h_out, int32_t out_kind);

/* tbk_predict for callers that may not allocate device memory while predicting (a server
 * whose memory budget is fixed at start-up, a latency-critical loop that cannot risk the
 * synchronisation an allocation can imply, a runtime that forbids allocations outside its
 * own pool).  It has no counterpart in the reference.  Same arguments, same results as
 * tbk_predict, computed by the same two kernels (walk into per-tree-chunk partial sums,
 * atomic-free second pass), but the partial sums live in a fixed 8 MiB array inside the
 * library image instead of a buffer grown with cudaMalloc; the call performs no
 * cudaMalloc / cudaFree and uses no allocating library.
 *   - Limit: n_rows x tree chunks x max(1, num_classes) <= 2 Mi (2097152) floats; larger
 *     requests fail with TBK_ERR_UNSUPPORTED and a message naming the sizes.  Split the
 *     batch, pin tree_chunks in the schedule, or use tbk_predict.
 *   - Every GPU that loads the library holds the array until the process exits.
 *   - The first call on a device looks up the array's device address (once per device);
 *     make that first call before any stream capture.
 *   - All calls on a device share the array: calls that overlap on the GPU (different
 *     streams, or different forests) race on it.  Serialise them.  Nothing in it needs
 *     clearing between calls: every element read by the second pass is written by the walk
 *     of the same call.
 *   - Forests in a 16-bit key layout (wide rows, deep trees) are not covered
 *     (TBK_ERR_UNSUPPORTED). */
TBK_EXPORT int tbk_predict_noalloc(tbk_forest *forest, const float *d_rows, int64_t n_rows, int64_t ld,
                                   void *d_out, int32_t out_kind, void *stream);

/* Device time of the walk (+ second pass) of the most recent tbk_predict* call on
 * this forest, in microseconds, measured with CUDA events when enabled; the
 * reference's counterpart is a host clock around the launch
 * (src/gpu/GPUSupportUtils.cpp:66-104, src/debug-helpers/TreePrintRoutines.cpp:203-220). */
TBK_EXPORT int tbk_set_timing(tbk_forest *forest, int32_t enable);
TBK_EXPORT int64_t tbk_last_kernel_time_us(tbk_forest *forest);

/* Reads the device status word (synchronises with the device): TBK_ERR_DEVICE_WAIT if
 * a bounded wait inside a kernel expired since the last check, else TBK_OK. */
TBK_EXPORT int tbk_check_status(tbk_forest *forest);

/* Failure drill, for tests of the error path: in the next tbk_predict* launch on this forest the
 * bulk copy of the first tree stage is never issued and the stage waits give up after a few
 * thousand polls, so the launch ends by itself with the status word set -- nothing faults or
 * hangs, the results of that launch are undefined, tbk_check_status() then returns
 * TBK_ERR_DEVICE_WAIT and the forest stays usable.  (The reference has no counterpart: its
 * generated kernels have no waits and its host code aborts on errors.)  A launch that stages
 * no trees (cache_trees = 2) has no such wait and is not affected. */
TBK_EXPORT int tbk_debug_expire_next_wait(tbk_forest *forest);

/* Number of kernel launches issued on behalf of this forest since creation. */
TBK_EXPORT int64_t tbk_launch_count(const tbk_forest *forest);

/* Host-only check of the forest-to-buffer lowering: packs the forest exactly as
 * tbk_forest_create would and interprets the packed buffers on the CPU with the slot
 * arithmetic the kernels use.  leaf_ids (n_rows x num_trees) and sums
 * (n_rows x max(1, num_classes)) may be NULL; rows may be NULL to pack only.  info, when
 * given, receives sizes (reserved[0] = tile shapes, reserved[1] = look-up-table bytes,
 * reserved[2] = bytes of the largest tree group).  No device is touched and no
 * prediction entry point uses this routine: it exists for the layout known-answer
 * tests that the reference runs on its serialised buffers (src/test/TestMain.cpp:903-1129). */
TBK_EXPORT int tbk_host_layout_check(const tbk_forest_arrays *forest, const tbk_schedule *schedule,
                                     const float *rows, int64_t n_rows, int64_t ld, int32_t *leaf_ids,
                                     float *sums, tbk_forest_info *info);

/* Host-only view of the launch-shape selector for a forest of the given shape (what the
 * reference's auto-scheduler decides in src/mlir/GPUAutoSchedule.cpp:318-472).  info
 * receives the schedule, shared-memory bytes and threads per block (reserved[0] = rows
 * cached in shared memory, reserved[1] = grid.x, reserved[2] = groups per tree chunk,
 * reserved[3] = 1 when class sums stay in registers, i.e. the block has no class table).
 * partial_sums != 0 asks for the plan of a launch that writes per-row partial sums
 * (tbk_predict_partial, tbk_predict_noalloc) instead of predictions. */
TBK_EXPORT int tbk_plan_launch(int32_t num_features, int32_t num_classes, int64_t num_groups,
                               int64_t max_group_bytes, int32_t lut_bytes, const tbk_schedule *schedule,
                               int64_t n_rows, int32_t smem_limit, int32_t num_sms, int32_t partial_sums,
                               tbk_forest_info *info);

TBK_EXPORT const char *tbk_last_error(void);

#ifdef __cplusplus
}
#endif
#endif /* TBK_H */
