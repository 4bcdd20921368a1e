/*
 * tbruntime.h -- the compile-then-run inference-runner API, with the entry-point names
 * and C signatures of the reference's libtreebeard-runtime.so (src/runtime/tbruntime.h:10-48
 * and the extern "C" definitions in src/runtime/runtime.cpp), which its ctypes binding
 * (src/python/treebeard_runtime_api.py:15-280) loads by name.  Handles are opaque and
 * travel as intptr_t / void*, exactly as there.
 *
 * Differences, all additive:
 *   - nothing aborts: a failing call returns 0 / does nothing and records a status and a
 *     message readable through TB_GetLastStatus / TB_GetLastError;
 *   - there is one back end (the B200 kernels): the CPU-runner constructors build the
 *     same GPU runner, and the entry points that emit LLVM IR write a compiled-model
 *     file instead (binary forest + bound options), which InitializeInferenceRunner loads;
 *   - RunInference accepts host pointers (as the reference) and CUDA device pointers.
 */
#ifndef TBRUNTIME_H
#define TBRUNTIME_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#else
#include <stdbool.h>
#endif

#define TREEBEARD_RUNTIME_EXPORT __attribute__((visibility("default")))

/* ---- execution (src/runtime/runtime.cpp:35-121) ---- */
/* Builds a runner from a compiled-model file written by GenerateLLVMIRForXGBoostModel /
 * CreateLLVMIRForONNXModel / LowerToLLVMAndDumpIR -- the counterpart of the reference's
 * ahead-of-time .so + globals JSON pair (runtime.cpp:35-54).  modelGlobalsJSONPath may be
 * NULL or empty; when given, the options it names replace those stored in the file. */
TREEBEARD_RUNTIME_EXPORT intptr_t InitializeInferenceRunner(const char *modelFilePath,
                                                            const char *modelGlobalsJSONPath);
/* inputs: batchSize x rowSize fp32, row-major; results: batchSize elements of the
 * return type (fp32, or int8 class ids) -- runtime.cpp:58-67 */
TREEBEARD_RUNTIME_EXPORT void RunInference(intptr_t inferenceRunner, void *inputs, void *results);
/* numRows must be a multiple of the batch size -- runtime.cpp:69-92 */
TREEBEARD_RUNTIME_EXPORT void RunInferenceOnMultipleBatches(intptr_t inferenceRunner, void *inputs,
                                                            void *results, int32_t numRows);
TREEBEARD_RUNTIME_EXPORT int32_t GetBatchSize(intptr_t inferenceRunner); /* runtime.cpp:94 */
TREEBEARD_RUNTIME_EXPORT int32_t GetRowSize(intptr_t inferenceRunner);   /* runtime.cpp:103 */
TREEBEARD_RUNTIME_EXPORT void DeleteInferenceRunner(intptr_t inferenceRunner); /* :112 */

/* ---- compiler options (runtime.cpp:123-174; fields src/include/TreebeardContext.h:64-136) ---- */
TREEBEARD_RUNTIME_EXPORT intptr_t CreateCompilerOptions(void);
TREEBEARD_RUNTIME_EXPORT void DeleteCompilerOptions(intptr_t options);
TREEBEARD_RUNTIME_EXPORT void Set_numberOfFeatures(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_batchSize(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_tileSize(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_thresholdTypeWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_returnTypeWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_returnTypeFloatType(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_featureIndexTypeWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_nodeIndexTypeWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_inputElementTypeWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_tileShapeBitWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_childIndexBitWidth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_makeAllLeavesSameDepth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_reorderTreesByDepth(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_statsProfileCSVPath(intptr_t options, const char *val);
TREEBEARD_RUNTIME_EXPORT void Set_pipelineSize(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_numberOfCores(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_numParallelTreeBatches(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_tilingType(intptr_t options, int32_t val); /* runtime.cpp:161 */

/* ---- GPU auto-schedule options (runtime.cpp:181-208; TreebeardContext.h:138-162) ---- */
TREEBEARD_RUNTIME_EXPORT intptr_t CreateGPUAutoScheduleOptions(void);
TREEBEARD_RUNTIME_EXPORT void DeleteGPUAutoScheduleOptions(intptr_t options);
TREEBEARD_RUNTIME_EXPORT void Set_numRowsPerTB(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_numRowsPerThread(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_rowTileSize(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_numTreeThreads(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_numTreesAtATime(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_cacheRows(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_cacheTrees(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_unrollTreeWalks(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_treeWalkInterleaveFactor(intptr_t options, int32_t val);
TREEBEARD_RUNTIME_EXPORT void Set_sharedMemoryReduce(intptr_t options, int32_t val);

/* ---- one-call runner construction (runtime.cpp:216-297) ---- */
/* The two "LLVM IR" calls write the compiled-model file to their second path and the
 * globals JSON to their third (there is no LLVM back end). */
TREEBEARD_RUNTIME_EXPORT void GenerateLLVMIRForXGBoostModel(const char *modelJSONPath, const char *llvmIRPath,
                                                            const char *modelGlobalsJSONPath, intptr_t options);
TREEBEARD_RUNTIME_EXPORT intptr_t CreateInferenceRunner(const char *modelJSONPath, const char *profileCSVPath,
                                                        intptr_t options);
TREEBEARD_RUNTIME_EXPORT void CreateLLVMIRForONNXModel(const char *modelPath, const char *llvmIRPath,
                                                       const char *modelGlobalsJSONPath, intptr_t options);
TREEBEARD_RUNTIME_EXPORT intptr_t CreateInferenceRunnerForONNXModel(const char *modelPath, intptr_t options);

/* ---- process-wide switches (runtime.cpp:301-325) ---- */
TREEBEARD_RUNTIME_EXPORT void SetEnableSparseRepresentation(int32_t val);
TREEBEARD_RUNTIME_EXPORT int32_t IsSparseRepresentationEnabled(void);
TREEBEARD_RUNTIME_EXPORT void SetPeeledCodeGenForProbabilityBasedTiling(int32_t val);
TREEBEARD_RUNTIME_EXPORT int32_t IsPeeledCodeGenForProbabilityBasedTilingEnabled(void);
TREEBEARD_RUNTIME_EXPORT void SetEnableMeasureGpuKernelTime(bool val);
TREEBEARD_RUNTIME_EXPORT void SetNumberOfKernelRuns(int32_t val);

/* ---- representation objects (runtime.cpp:340-358) ---- */
TREEBEARD_RUNTIME_EXPORT void *ConstructRepresentation(const char *repName);
TREEBEARD_RUNTIME_EXPORT void DestroyRepresentation(void *rep);

/* ---- context (runtime.cpp:363-416) ---- */
TREEBEARD_RUNTIME_EXPORT intptr_t ConstructTreebeardContext(const char *modelPath, const char *modelGlobalsJSONPath,
                                                            intptr_t options);
TREEBEARD_RUNTIME_EXPORT intptr_t ConstructTreebeardContextFromGPUAutoscheduleOptions(
    const char *modelPath, const char *modelGlobalsJSONPath, intptr_t options, intptr_t gpuScheduleOptions);
TREEBEARD_RUNTIME_EXPORT void DestroyTreebeardContext(intptr_t tbContext);
/* "xgboost_json" or "onnx_file" (src/json/ForestCreatorFactory.cpp:7-11) */
TREEBEARD_RUNTIME_EXPORT void SetForestCreatorType(intptr_t tbContext, const char *creatorType);
/* "gpu_array", "gpu_sparse", "gpu_reorg", "array", "sparse"; addition: "gpu_auto" lets the
 * library choose the layout for the forest (what findBestGPUScheduleAndCompileModel uses) */
TREEBEARD_RUNTIME_EXPORT void SetRepresentationAndSerializer(intptr_t tbContext, const char *repType);
TREEBEARD_RUNTIME_EXPORT void *GetScheduleFromTBContext(intptr_t tbContext);

/* ---- compilation (runtime.cpp:418-478, 769-798) ---- */
TREEBEARD_RUNTIME_EXPORT void BuildHIRRepresentation(void *tbContext);
TREEBEARD_RUNTIME_EXPORT bool LowerToLLVMAndDumpIR(void *tbContext, const char *fileName);
TREEBEARD_RUNTIME_EXPORT void *ConstructInferenceRunnerFromHIR(void *tbContext);
TREEBEARD_RUNTIME_EXPORT void *ConstructGPUInferenceRunnerFromHIR(void *tbContext);
TREEBEARD_RUNTIME_EXPORT void *ConstructGPUInferenceRunnerFromTBContext(void *tbContext);
TREEBEARD_RUNTIME_EXPORT void *findBestGPUScheduleAndCompileModel(void *tbContext);
TREEBEARD_RUNTIME_EXPORT void SetOneTreeAtATimeSchedule(intptr_t options); /* runtime.cpp:486 */

/* ---- schedule objects (runtime.cpp:500-750).  The kernel family is fixed: directives
 * are recorded, reported by Schedule_PrintToString and otherwise have no effect; the
 * launch shape comes from the GPU auto-schedule options and the selector. ---- */
TREEBEARD_RUNTIME_EXPORT intptr_t Schedule_NewIndexVariable(intptr_t schedPtr, const char *name);
TREEBEARD_RUNTIME_EXPORT intptr_t Schedule_NewIndexVariable2(intptr_t schedPtr, intptr_t indexVarPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_Tile(intptr_t schedPtr, intptr_t indexPtr, intptr_t outerPtr,
                                            intptr_t innerPtr, int32_t tileSize);
TREEBEARD_RUNTIME_EXPORT void Schedule_Reorder(intptr_t schedPtr, intptr_t indicesPtr, int32_t numIndices);
TREEBEARD_RUNTIME_EXPORT void Schedule_Split(intptr_t schedPtr, intptr_t indexPtr, intptr_t firstPtr,
                                             intptr_t secondPtr, int32_t splitIteration, intptr_t indexMapPtr);
TREEBEARD_RUNTIME_EXPORT intptr_t Schedule_Specialize(intptr_t schedPtr, intptr_t indexPtr);
TREEBEARD_RUNTIME_EXPORT int64_t GetSpecializationInfoNumIterations(intptr_t infoPtr);
TREEBEARD_RUNTIME_EXPORT int64_t GetSpecializationInfoNumEntries(intptr_t infoPtr);
TREEBEARD_RUNTIME_EXPORT void GetSpecializationInfoEntries(intptr_t infoPtr, intptr_t lengths, intptr_t indices);
TREEBEARD_RUNTIME_EXPORT void Schedule_Pipeline(intptr_t schedPtr, intptr_t indexPtr, int32_t stepSize);
TREEBEARD_RUNTIME_EXPORT void Schedule_Simdize(intptr_t schedPtr, intptr_t indexPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_Parallel(intptr_t schedPtr, intptr_t indexPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_Unroll(intptr_t schedPtr, intptr_t indexVarPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_PeelWalk(intptr_t schedPtr, intptr_t indexVarPtr, int32_t numberOfIterations);
TREEBEARD_RUNTIME_EXPORT void Schedule_Cache(intptr_t schedPtr, intptr_t indexVarPtr);
TREEBEARD_RUNTIME_EXPORT intptr_t Schedule_GetRootIndex(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT intptr_t Schedule_GetBatchIndex(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT intptr_t Schedule_GetTreeIndex(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT int32_t Schedule_PrintToString(intptr_t schedPtr, intptr_t str, int32_t strLen);
TREEBEARD_RUNTIME_EXPORT int32_t Schedule_GetBatchSize(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT int32_t Schedule_GetForestSize(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT bool Schedule_IsDefaultSchedule(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_Finalize(intptr_t schedPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_AtomicReduce(intptr_t schedPtr, intptr_t indexVarPtr);
TREEBEARD_RUNTIME_EXPORT void Schedule_VectorReduce(intptr_t schedPtr, intptr_t indexVarPtr, int32_t width);
TREEBEARD_RUNTIME_EXPORT void Schedule_SharedReduce(intptr_t schedPtr, intptr_t indexVarPtr);
TREEBEARD_RUNTIME_EXPORT void IndexVariable_SetGPUThreadDim(intptr_t indexVarPtr, int32_t construct, int32_t dim);

/* Accumulated device time of the walk kernels of this runner in microseconds, when
 * SetEnableMeasureGpuKernelTime(true) was in force (runtime.cpp:753-758). */
TREEBEARD_RUNTIME_EXPORT int64_t GetGPUKernelExecutionTime(intptr_t inferenceRunner);

/* ---- additions (no counterpart in the reference) ---- */
TREEBEARD_RUNTIME_EXPORT int32_t TB_GetLastStatus(void);
TREEBEARD_RUNTIME_EXPORT const char *TB_GetLastError(void);
/* CUDA device the next runner is built on (default 0). */
TREEBEARD_RUNTIME_EXPORT void TB_SetDevice(int32_t device);
/* Several devices for the next runner: it keeps a copy of the forest on each, cuts every HOST
 * batch (RunInference / RunInferenceOnMultipleBatches) into one contiguous row range per device
 * and predicts them concurrently; device-resident batches run on the first device. */
TREEBEARD_RUNTIME_EXPORT void TB_SetDevices(const int32_t *devices, int32_t count);
TREEBEARD_RUNTIME_EXPORT int32_t TB_RunnerDeviceCount(intptr_t inferenceRunner);
/* The kernel-level forest handle (tbk_forest*, include/tbk.h) behind a runner, for
 * callers that hold device-resident inputs. */
TREEBEARD_RUNTIME_EXPORT void *TB_GetKernelForest(intptr_t inferenceRunner);
/* Builds a runner directly from flat forest arrays (tbk_forest_arrays*, include/tbk.h). */
TREEBEARD_RUNTIME_EXPORT intptr_t TB_CreateInferenceRunnerFromArrays(const void *forestArrays, intptr_t options,
                                                                     intptr_t gpuScheduleOptions,
                                                                     const char *representation);
/* Host-side model loading, no device involved: parses a model file with the named front
 * end ("xgboost_json" / "onnx_file", or "compiled_model" for a compiled-model file; numberOfFeatures as in Set_numberOfFeatures, 0 = from
 * the file) and exposes the forest as flat arrays (tbk_forest_arrays*, include/tbk.h; the
 * pointers stay valid until TB_FreeForest).  What the reference's ForestCreator builds in
 * ConstructForest (src/json/xgboostparser.h:116-219, src/json/onnxmodelparser.h:220-374). */
TREEBEARD_RUNTIME_EXPORT intptr_t TB_LoadForest(const char *modelPath, const char *creatorType,
                                                int32_t numberOfFeatures);
TREEBEARD_RUNTIME_EXPORT int32_t TB_ForestGetArrays(intptr_t forest, void *forestArraysOut);
TREEBEARD_RUNTIME_EXPORT void TB_FreeForest(intptr_t forest);
/* Width in bits of the input element / result element types of a runner
 * (GetInputTypeBitWidth / GetReturnTypeBitWidth of the generated module,
 * src/json/forestcreator.h:307-313). */
/* 1 if the runner was built from the packed image cached in a compiled-model file (the packer
 * did not run), 0 if the forest was packed afresh. */
TREEBEARD_RUNTIME_EXPORT int32_t TB_RunnerUsedPackedImage(intptr_t inferenceRunner);
TREEBEARD_RUNTIME_EXPORT int32_t TB_GetInputTypeBitWidth(intptr_t inferenceRunner);
TREEBEARD_RUNTIME_EXPORT int32_t TB_GetReturnTypeBitWidth(intptr_t inferenceRunner);

#ifdef __cplusplus
}
#endif
#endif /* TBRUNTIME_H */
