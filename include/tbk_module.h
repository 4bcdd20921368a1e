/*
 * tbk_module.h -- the module-side symbols of the reference's inference runner, on top of the
 * B200 kernels: a shared library (libtbk_module.so) that exports what the reference's runner
 * resolves BY NAME in a compiled module -- Prediction_Function, Init_Model, Init_Offsets,
 * Init_Lengths, Init_ClassIds, Dealloc_Buffers, GetBatchSize, GetRowSize,
 * GetInputTypeBitWidth, GetReturnTypeBitWidth (src/mlir/ExecutionHelpers.cpp:37-51, 78-94
 * for the dlsym look-up; src/gpu/GPUModelSerializers.cpp:21-262 for the calls) -- with the
 * calling convention of MLIR's expanded memref descriptors: a rank-1 memref travels as five
 * arguments (base pointer, aligned pointer, offset, size, stride), a rank-2 memref as seven,
 * and a memref result is returned by value (src/mlir/TypeDefinitions.h:10-17).
 *
 * Covered: scalar tiles (tile size 1) of the array and the sparse representation
 * (libtbk_module.so) and of the reorg representation (libtbk_module_reorg.so: the same
 * names, but Init_Thresholds / Init_FeatureIndices instead of Init_Model / Init_Offsets /
 * Init_Lengths, and other arguments to Prediction_Function and Dealloc_Buffers,
 * src/gpu/ReorgForestRepresentation.cpp:278-377; include this header with TBK_MODULE_REORG
 * defined for its declarations); fp32 thresholds, 8-, 16- or 32-bit feature indices, 16- or
 * 32-bit child indices, fp32 inputs, fp32 or (multiclass) int8 results.  In the reference a module is generated for ONE model and has batch size,
 * row size, initial value, transformation and class count compiled in; this library is
 * generic, so the host states them once with TBK_Module_Configure before the Init_* calls.
 * One model per loaded library, like a compiled module.
 *
 * Init_Model receives the serializer's buffers (src/include/DecisionForest.h:292-315 array
 * layout: a complete array per tree, leaf = feature index -1 with the value in the threshold;
 * :595-629 sparse layout: level order, child index = left child, right child = left + 1) and
 * rebuilds the forest from them.  The reorg buffers (src/gpu/ReorgForestRepresentation.cpp:
 * 186-211, 258-276) hold slot s of tree t at s * num_trees + t, every tree a complete array of
 * the deepest tree's 2^depth - 1 slots, unused slots with feature index -1; the tree count is
 * compiled into a reference module and comes from the configuration here.  Prediction_Function
 * takes HOST memrefs and runs the chunked
 * copy-in / walk / copy-out pipeline (tbk_predict_host).
 */
#ifndef TBK_MODULE_H
#define TBK_MODULE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TBK_MODULE_EXPORT __attribute__((visibility("default")))

/* rank-1 memref as the reference declares it (src/mlir/TypeDefinitions.h:10-17) */
typedef struct tbk_memref1 {
  void *bufferPtr;
  void *alignedPtr;
  int64_t offset;
  int64_t lengths[1];
  int64_t strides[1];
} tbk_memref1;

typedef struct tbk_module_config {
  int32_t batch_size;          /* rows per Prediction_Function call */
  int32_t row_size;            /* features per row */
  int32_t sparse;              /* 1: Init_Model also receives child indices */
  int32_t feature_index_width; /* 16 or 32 */
  int32_t child_index_width;   /* 16 or 32 (sparse) */
  int32_t tile_shape_width;    /* 8, 16 or 32: only skipped over, tile size is 1 */
  int32_t num_classes;         /* 0 = single output */
  int32_t transform;           /* TBK_IDENTITY / TBK_SIGMOID / TBK_SOFTMAX (include/tbk.h) */
  int32_t return_width;        /* 32 (fp32) or 8 (int8 class id) */
  int32_t device;
  int32_t num_trees;           /* reorg only: trees interleaved in the two buffers */
  int32_t reserved;
  double initial_value;
} tbk_module_config;

/* no counterpart in the reference (see above); 0 = ok */
TBK_MODULE_EXPORT int32_t TBK_Module_Configure(const tbk_module_config *config);
TBK_MODULE_EXPORT const char *TBK_Module_LastError(void);

/* src/mlir/ExecutionHelpers.cpp:37-51 */
TBK_MODULE_EXPORT int32_t GetBatchSize(void);
TBK_MODULE_EXPORT int32_t GetRowSize(void);
TBK_MODULE_EXPORT int32_t GetInputTypeBitWidth(void);
TBK_MODULE_EXPORT int32_t GetReturnTypeBitWidth(void);

/* src/gpu/GPUModelSerializers.cpp:184-202, src/gpu/ReorgForestRepresentation.cpp:313-318 */
TBK_MODULE_EXPORT tbk_memref1 Init_ClassIds(int8_t *base, int8_t *aligned, int64_t offset, int64_t size, int64_t stride);

#ifndef TBK_MODULE_REORG
/* src/gpu/GPUModelSerializers.cpp:21-59: (int64 memref) -> int64 memref */
TBK_MODULE_EXPORT tbk_memref1 Init_Lengths(int64_t *base, int64_t *aligned, int64_t offset, int64_t size, int64_t stride);
TBK_MODULE_EXPORT tbk_memref1 Init_Offsets(int64_t *base, int64_t *aligned, int64_t offset, int64_t size, int64_t stride);
/* :93-150: thresholds, feature indices, tile-shape ids [, child indices (sparse)] -> model */
TBK_MODULE_EXPORT tbk_memref1 Init_Model(void *thr, void *thrAligned, int64_t thrOffset, int64_t thrSize, int64_t thrStride,
                                         void *feat, void *featAligned, int64_t featOffset, int64_t featSize, int64_t featStride,
                                         void *shape, void *shapeAligned, int64_t shapeOffset, int64_t shapeSize, int64_t shapeStride,
                                         void *child, void *childAligned, int64_t childOffset, int64_t childSize, int64_t childStride);
/* :210-229: inputs (rank 2), results, model, offsets, lengths, class ids -> results */
TBK_MODULE_EXPORT tbk_memref1 Prediction_Function(
    void *in, void *inAligned, int64_t inOffset, int64_t inRows, int64_t inCols, int64_t inStride0, int64_t inStride1,
    void *out, void *outAligned, int64_t outOffset, int64_t outSize, int64_t outStride,
    void *model, void *modelAligned, int64_t modelOffset, int64_t modelSize, int64_t modelStride,
    int64_t *offsets, int64_t *offsetsAligned, int64_t offsetsOffset, int64_t offsetsSize, int64_t offsetsStride,
    int64_t *lengths, int64_t *lengthsAligned, int64_t lengthsOffset, int64_t lengthsSize, int64_t lengthsStride,
    int8_t *classIds, int8_t *classIdsAligned, int64_t classIdsOffset, int64_t classIdsSize, int64_t classIdsStride);
/* :231-262 (the class-id memref is passed only for multiclass models) */
TBK_MODULE_EXPORT int32_t Dealloc_Buffers(
    void *model, void *modelAligned, int64_t modelOffset, int64_t modelSize, int64_t modelStride,
    int64_t *offsets, int64_t *offsetsAligned, int64_t offsetsOffset, int64_t offsetsSize, int64_t offsetsStride,
    int64_t *lengths, int64_t *lengthsAligned, int64_t lengthsOffset, int64_t lengthsSize, int64_t lengthsStride);
#else
/* src/gpu/ReorgForestRepresentation.cpp:278-311: one buffer per call */
TBK_MODULE_EXPORT tbk_memref1 Init_Thresholds(float *base, float *aligned, int64_t offset, int64_t size, int64_t stride);
TBK_MODULE_EXPORT tbk_memref1 Init_FeatureIndices(void *base, void *aligned, int64_t offset, int64_t size, int64_t stride);
/* :321-348: inputs (rank 2), results, thresholds, feature indices, class ids -> results */
TBK_MODULE_EXPORT tbk_memref1 Prediction_Function(
    void *in, void *inAligned, int64_t inOffset, int64_t inRows, int64_t inCols, int64_t inStride0, int64_t inStride1,
    void *out, void *outAligned, int64_t outOffset, int64_t outSize, int64_t outStride,
    void *thr, void *thrAligned, int64_t thrOffset, int64_t thrSize, int64_t thrStride,
    void *feat, void *featAligned, int64_t featOffset, int64_t featSize, int64_t featStride,
    int8_t *classIds, int8_t *classIdsAligned, int64_t classIdsOffset, int64_t classIdsSize, int64_t classIdsStride);
/* :352-377 (a multiclass module is handed the class-id memref as well) */
TBK_MODULE_EXPORT int32_t Dealloc_Buffers(
    void *thr, void *thrAligned, int64_t thrOffset, int64_t thrSize, int64_t thrStride,
    void *feat, void *featAligned, int64_t featOffset, int64_t featSize, int64_t featStride);
#endif

#ifdef __cplusplus
}
#endif
#endif /* TBK_MODULE_H */
