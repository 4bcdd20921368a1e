"""Object wrapper over the inference-runner API: the classes and method names a user of
the reference's Python package (src/python/treebeard.py:11-410) already knows --
``CompilerOptions``, ``GPUAutoScheduleOptions``, ``TreebeardContext``,
``TreebeardInferenceRunner``, ``Schedule``/``IndexVariable`` -- bound to the B200
runtime.  ``RunInference`` takes a numpy array (host memory, as in the reference) or a
torch CUDA tensor (no copies)."""
import ctypes
from enum import Enum
from typing import List

import numpy

from .treebeard_runtime_api import TreebeardAPI, TreebeardRuntimeError  # noqa: F401

treebeardAPI = TreebeardAPI()
_rt = treebeardAPI.runtime_lib


class GPUAutoScheduleOptions:
    def __init__(self) -> None:
        self.optionsPtr = _rt.CreateGPUAutoScheduleOptions()
        self.unrollTreeWalks = False

    def __del__(self):
        _rt.DeleteGPUAutoScheduleOptions(self.optionsPtr)

    def NumberOfRowsPerThreadBlock(self, val: int):
        _rt.Set_numRowsPerTB(self.optionsPtr, val)

    def NumberOfRowsPerThread(self, val: int):
        _rt.Set_numRowsPerThread(self.optionsPtr, val)

    def RowTileSize(self, val: int):
        _rt.Set_rowTileSize(self.optionsPtr, val)

    def NumberOfTreeThreads(self, val: int):
        _rt.Set_numTreeThreads(self.optionsPtr, val)

    def NumberOfTreesAtATime(self, val: int):
        _rt.Set_numTreesAtATime(self.optionsPtr, val)

    def CacheRows(self, val: bool):
        _rt.Set_cacheRows(self.optionsPtr, int(bool(val)))

    def CacheTrees(self, val: bool):
        _rt.Set_cacheTrees(self.optionsPtr, int(bool(val)))

    def UnrollTreeWalks(self, val: bool):
        self.unrollTreeWalks = val
        _rt.Set_unrollTreeWalks(self.optionsPtr, int(bool(val)))

    def TreeWalkInterleaveFactor(self, val: int):
        _rt.Set_treeWalkInterleaveFactor(self.optionsPtr, val)

    def SharedReduce(self, val: bool):
        _rt.Set_sharedMemoryReduce(self.optionsPtr, int(bool(val)))

    @classmethod
    def Construct(cls, num_rows_per_TB: int, num_rows_per_thread: int = 1, num_tree_threads: int = 1,
                  cache_rows: bool = False, cache_trees: bool = False,
                  unroll_tree_walks: bool = False, tree_walk_interleave_factor: int = -1,
                  shared_reduce: bool = False):
        options = cls()
        options.NumberOfRowsPerThreadBlock(num_rows_per_TB)
        options.NumberOfRowsPerThread(num_rows_per_thread)
        options.RowTileSize(1)
        options.NumberOfTreeThreads(num_tree_threads)
        options.NumberOfTreesAtATime(1)
        options.CacheRows(cache_rows)
        options.CacheTrees(cache_trees)
        options.UnrollTreeWalks(unroll_tree_walks)
        options.TreeWalkInterleaveFactor(tree_walk_interleave_factor)
        options.SharedReduce(shared_reduce)
        return options


class CompilerOptions:
    def __init__(self, batchSize, tileSize) -> None:
        self.optionsPtr = _rt.CreateCompilerOptions()
        _rt.Set_batchSize(self.optionsPtr, batchSize)
        _rt.Set_tileSize(self.optionsPtr, tileSize)

    def __del__(self):
        _rt.DeleteCompilerOptions(self.optionsPtr)

    def SetThresholdTypeWidth(self, val: int):
        _rt.Set_thresholdTypeWidth(self.optionsPtr, val)

    def SetReturnTypeWidth(self, val: int):
        _rt.Set_returnTypeWidth(self.optionsPtr, val)

    def SetReturnTypeIsFloatType(self, val):
        _rt.Set_returnTypeFloatType(self.optionsPtr, int(bool(val)))

    def SetFeatureIndexTypeWidth(self, val: int):
        _rt.Set_featureIndexTypeWidth(self.optionsPtr, val)

    def SetNodeIndexTypeWidth(self, val: int):
        _rt.Set_nodeIndexTypeWidth(self.optionsPtr, val)

    def SetInputElementTypeWidth(self, val: int):
        _rt.Set_inputElementTypeWidth(self.optionsPtr, val)

    def SetTileShapeBitWidth(self, val: int):
        _rt.Set_tileShapeBitWidth(self.optionsPtr, val)

    def SetChildIndexBitWidth(self, val: int):
        _rt.Set_childIndexBitWidth(self.optionsPtr, val)

    def SetMakeAllLeavesSameDepth(self, val: int):
        _rt.Set_makeAllLeavesSameDepth(self.optionsPtr, val)

    def SetReorderTreesByDepth(self, val):
        _rt.Set_reorderTreesByDepth(self.optionsPtr, int(bool(val)))

    def SetTilingType(self, val: int):
        _rt.Set_tilingType(self.optionsPtr, val)

    def SetPipelineWidth(self, val: int):
        _rt.Set_pipelineSize(self.optionsPtr, val)

    def SetNumberOfFeatures(self, val: int):
        _rt.Set_numberOfFeatures(self.optionsPtr, val)

    def SetNumberOfCores(self, val: int):
        _rt.Set_numberOfCores(self.optionsPtr, val)

    def SetStatsProfileCSVPath(self, val: str):
        _rt.Set_statsProfileCSVPath(self.optionsPtr, val.encode("ascii"))

    def SetOneTreeAtATimeSchedule(self):
        _rt.SetOneTreeAtATimeSchedule(self.optionsPtr)

    def SetNumberOfParallelTreeBatches(self, val: int):
        _rt.Set_numParallelTreeBatches(self.optionsPtr, val)


class GPUConstruct(Enum):
    Grid = 0
    ThreadBlock = 1
    Undef = 2


class Dimension(Enum):
    X = 0
    Y = 1
    Z = 2


class IndexVariable:
    def __init__(self, name, indexVarPtr) -> None:
        self.name = name
        self.indexVarPtr = indexVarPtr

    def set_gpu_dimension(self, gpuConstruct: GPUConstruct, dimension: Dimension):
        _rt.IndexVariable_SetGPUThreadDim(self.indexVarPtr, gpuConstruct.value, dimension.value)


class Schedule:
    """Loop-nest directives.  They are recorded and printable; the launch shape of the
    fixed kernel family comes from GPUAutoScheduleOptions and the selector."""

    def __init__(self, schedulePtr):
        self.schedulePtr = schedulePtr

    def NewIndexVariable(self, name):
        return IndexVariable(name, _rt.Schedule_NewIndexVariable(self.schedulePtr, name.encode("ascii")))

    def Tile(self, index, outerIndex, innerIndex, tileSize):
        _rt.Schedule_Tile(self.schedulePtr, index.indexVarPtr, outerIndex.indexVarPtr,
                          innerIndex.indexVarPtr, tileSize)

    def Reorder(self, indices: List[IndexVariable]):
        arr = numpy.array([i.indexVarPtr for i in indices], numpy.int64)
        _rt.Schedule_Reorder(self.schedulePtr, arr.ctypes.data_as(ctypes.c_void_p), len(indices))

    def Specialize(self, index):
        _rt.Schedule_Specialize(self.schedulePtr, index.indexVarPtr)
        return []

    def Pipeline(self, index, stepSize):
        _rt.Schedule_Pipeline(self.schedulePtr, index.indexVarPtr, stepSize)

    def Simdize(self, index):
        _rt.Schedule_Simdize(self.schedulePtr, index.indexVarPtr)

    def Parallel(self, index):
        _rt.Schedule_Parallel(self.schedulePtr, index.indexVarPtr)

    def Unroll(self, index):
        _rt.Schedule_Unroll(self.schedulePtr, index.indexVarPtr)

    def PeelWalk(self, index, numberOfIterations):
        _rt.Schedule_PeelWalk(self.schedulePtr, index.indexVarPtr, numberOfIterations)

    def Cache(self, index):
        _rt.Schedule_Cache(self.schedulePtr, index.indexVarPtr)

    def AtomicReduce(self, index):
        _rt.Schedule_AtomicReduce(self.schedulePtr, index.indexVarPtr)

    def VectorReduce(self, index, width):
        _rt.Schedule_VectorReduce(self.schedulePtr, index.indexVarPtr, width)

    def SharedReduce(self, index):
        _rt.Schedule_SharedReduce(self.schedulePtr, index.indexVarPtr)

    def GetRootIndex(self):
        return IndexVariable("root", _rt.Schedule_GetRootIndex(self.schedulePtr))

    def GetBatchIndex(self):
        return IndexVariable("batch", _rt.Schedule_GetBatchIndex(self.schedulePtr))

    def GetTreeIndex(self):
        return IndexVariable("tree", _rt.Schedule_GetTreeIndex(self.schedulePtr))

    def PrintToString(self) -> str:
        buf = ctypes.create_string_buffer(1 << 16)
        n = _rt.Schedule_PrintToString(self.schedulePtr, ctypes.addressof(buf), len(buf))
        return buf.value.decode() if n >= 0 else ""

    def GetBatchSize(self):
        return _rt.Schedule_GetBatchSize(self.schedulePtr)

    def GetForestSize(self):
        return _rt.Schedule_GetForestSize(self.schedulePtr)

    def IsDefaultSchedule(self):
        return _rt.Schedule_IsDefaultSchedule(self.schedulePtr)

    def Finalize(self):
        _rt.Schedule_Finalize(self.schedulePtr)


class TreebeardContext:
    def __init__(self, model_filepath: str, globals_file_path: str, options: CompilerOptions,
                 gpuAutoScheduleOptions: GPUAutoScheduleOptions = None) -> None:
        self._options = options  # keep alive
        if gpuAutoScheduleOptions is None:
            self.tbcontextPtr = treebeardAPI.ConstructTreebeardContext(
                model_filepath, globals_file_path, options.optionsPtr)
        else:
            self.tbcontextPtr = treebeardAPI.ConstructTreebeardContextFromGPUAutoscheduleOptions(
                model_filepath, globals_file_path, options.optionsPtr,
                gpuAutoScheduleOptions.optionsPtr)
        treebeardAPI.check()

    def __del__(self):
        treebeardAPI.DestroyTreebeardContext(self.tbcontextPtr)

    def SetInputFiletype(self, file_type: str) -> None:
        treebeardAPI.SetForestCreatorType(self.tbcontextPtr, file_type)

    def SetRepresentationType(self, rep_type: str) -> None:
        treebeardAPI.SetRepresentationAndSerializer(self.tbcontextPtr, rep_type)

    def GetSchedule(self):
        return Schedule(treebeardAPI.GetScheduleFromTBContext(self.tbcontextPtr))

    def BuildHIRRepresentation(self):
        _rt.BuildHIRRepresentation(self.tbcontextPtr)
        treebeardAPI.check()

    def DumpLLVMIR(self, path: str):
        treebeardAPI.LowerToLLVMAndDumpIR(self.tbcontextPtr, path)
        treebeardAPI.check()

    def _runner(self, ctor):
        return TreebeardInferenceRunner._wrap(int(ctor(self.tbcontextPtr) or 0))

    def ConstructInferenceRunnerFromHIR(self):
        return self._runner(_rt.ConstructInferenceRunnerFromHIR)

    def ConstructGPUInferenceRunnerFromHIR(self):
        return self._runner(_rt.ConstructGPUInferenceRunnerFromHIR)

    def ConstructGPUInferenceRunnerAutoSchedule(self):
        return self._runner(_rt.findBestGPUScheduleAndCompileModel)


class TreebeardInferenceRunner:
    def __init__(self) -> None:
        self.treebeardAPI = treebeardAPI
        self.inferenceRunner = 0
        self.rowSize = -1
        self.batchSize = -1

    @classmethod
    def _wrap(cls, handle: int):
        if not handle:
            treebeardAPI.check()
            raise TreebeardRuntimeError("runner construction failed")
        r = cls()
        r.inferenceRunner = handle
        r.rowSize = treebeardAPI.GetRowSize(handle)
        r.batchSize = treebeardAPI.GetBatchSize(handle)
        return r

    @classmethod
    def FromSOFile(cls, modelSOPath: str, modelGlobalsJSONPath: str):
        return cls._wrap(treebeardAPI.InitializeInferenceRunner(modelSOPath, modelGlobalsJSONPath))

    @classmethod
    def FromModelFile(cls, modelJSONPathStr: str, profileCSVPathStr: str, options: CompilerOptions):
        return cls._wrap(_rt.CreateInferenceRunner(modelJSONPathStr.encode("ascii"),
                                                   profileCSVPathStr.encode("ascii"),
                                                   options.optionsPtr))

    @classmethod
    def FromONNXModelFile(cls, onnx_model_path: str, options: CompilerOptions):
        return cls._wrap(_rt.CreateInferenceRunnerForONNXModel(onnx_model_path.encode("ascii"),
                                                               options.optionsPtr))

    @classmethod
    def FromTBContext(cls, tbContext):
        tbContext.BuildHIRRepresentation()
        return tbContext.ConstructInferenceRunnerFromHIR()

    @classmethod
    def GPUInferenceRunnerFromTBContext(cls, tbContext):
        return cls._wrap(int(_rt.ConstructGPUInferenceRunnerFromTBContext(tbContext.tbcontextPtr) or 0))

    @classmethod
    def AutoScheduleGPUInferenceRunnerFromTBContext(cls, tbContext):
        return tbContext.ConstructGPUInferenceRunnerAutoSchedule()

    @classmethod
    def FromForestArrays(cls, forest, options: CompilerOptions, representation: str = "gpu_sparse",
                         gpuAutoScheduleOptions: GPUAutoScheduleOptions = None):
        """Builds a runner from flat forest arrays (no model file)."""
        from .kernels import forest_arrays_c
        c, keep = forest_arrays_c(forest)
        gpu = gpuAutoScheduleOptions.optionsPtr if gpuAutoScheduleOptions is not None else 0
        return cls._wrap(_rt.TB_CreateInferenceRunnerFromArrays(
            ctypes.addressof(c), options.optionsPtr, gpu, representation.encode("ascii")))

    def __del__(self):
        if self.inferenceRunner:
            self.treebeardAPI.DeleteInferenceRunner(self.inferenceRunner)
            self.inferenceRunner = 0

    def _is_int8(self):
        return _rt.TB_GetReturnTypeBitWidth(self.inferenceRunner) == 8

    def _check_shape(self, inputs, rows):
        """The library reads rows x GetRowSize floats: a smaller buffer would be overrun."""
        shape = tuple(inputs.shape)
        ok = (len(shape) == 2 and shape[1] == self.rowSize and (rows is None or shape[0] == rows)) or \
             (len(shape) == 1 and rows is not None and shape[0] == rows * self.rowSize)
        if not ok:
            want = f"({rows if rows is not None else 'n'}, {self.rowSize})"
            raise TreebeardRuntimeError(f"inputs have shape {shape}, the runner expects {want}")

    def _host_types(self, resultType):
        """numpy types of the host buffers: what the runner was compiled for (32- or 64-bit
        inputs; fp32, fp64 or int8 results)."""
        in_type = numpy.float64 if _rt.TB_GetInputTypeBitWidth(self.inferenceRunner) == 64 else numpy.float32
        width = _rt.TB_GetReturnTypeBitWidth(self.inferenceRunner)
        out_type = numpy.int8 if width == 8 else numpy.float64 if width == 64 else numpy.float32
        if numpy.dtype(resultType) != numpy.dtype(out_type):
            raise TreebeardRuntimeError(f"the runner returns {numpy.dtype(out_type)}, not {numpy.dtype(resultType)}")
        return in_type, out_type

    def RunInference(self, inputs, resultType=numpy.float32):
        if isinstance(inputs, numpy.ndarray):
            in_type, resultType = self._host_types(resultType)
            assert inputs.dtype == in_type and inputs.flags.c_contiguous
            self._check_shape(inputs, self.batchSize)
            results = numpy.zeros((self.batchSize), resultType)
            self.treebeardAPI.RunInference(self.inferenceRunner, inputs.ctypes.data, results.ctypes.data)
            return results
        import torch  # device-resident path
        assert inputs.is_cuda and inputs.dtype == torch.float32 and inputs.is_contiguous()
        self._check_shape(inputs, self.batchSize)
        results = torch.zeros(self.batchSize, device=inputs.device,
                              dtype=torch.int8 if self._is_int8() else torch.float32)
        self.treebeardAPI.RunInference(self.inferenceRunner, inputs.data_ptr(), results.data_ptr())
        return results

    def RunInferenceOnMultipleBatches(self, inputs, resultType=numpy.float32):
        assert type(inputs) is numpy.ndarray
        in_type, resultType = self._host_types(resultType)
        assert inputs.dtype == in_type and inputs.flags.c_contiguous
        self._check_shape(inputs, None)
        numRows = inputs.shape[0]
        results = numpy.zeros((numRows), resultType)
        self.treebeardAPI.RunInferenceOnMultipleBatches(self.inferenceRunner, inputs.ctypes.data,
                                                        results.ctypes.data, numRows)
        return results

    def device_count(self) -> int:
        """Devices this runner spreads host batches over (see SetDevices)."""
        return int(_rt.TB_RunnerDeviceCount(self.inferenceRunner))

    def used_packed_image(self) -> bool:
        """True if this runner was built from the packed image cached in a compiled-model file."""
        return bool(_rt.TB_RunnerUsedPackedImage(self.inferenceRunner))

    def kernel_forest(self):
        """The kernel-level handle behind this runner (see kernels.DeviceForest)."""
        return int(_rt.TB_GetKernelForest(self.inferenceRunner) or 0)


def LoadForest(model_path: str, file_type: str = "xgboost_json", number_of_features: int = 0):
    """Parses a model file with the native front end ("xgboost_json" / "onnx_file") and
    returns the forest as flat numpy arrays (a ``synth.ForestArrays``).  Host only."""
    from .kernels import ForestArraysC
    from .synth import ForestArrays
    h = _rt.TB_LoadForest(model_path.encode("ascii"), file_type.encode("ascii"), number_of_features)
    if not h:
        treebeardAPI.check()
        raise TreebeardRuntimeError("model could not be loaded")
    try:
        c = ForestArraysC()
        _rt.TB_ForestGetArrays(h, ctypes.addressof(c))
        T = c.num_trees
        off = numpy.ctypeslib.as_array(ctypes.cast(c.tree_off, ctypes.POINTER(ctypes.c_int64)), (T + 1,)).copy()
        n = int(off[-1])

        def arr(ptr, ctype, count):
            return numpy.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctype)), (count,)).copy()
        return ForestArrays(off, arr(c.left, ctypes.c_int32, n), arr(c.right, ctypes.c_int32, n),
                            arr(c.feat, ctypes.c_int32, n), arr(c.thr, ctypes.c_float, n),
                            arr(c.class_id, ctypes.c_int32, T), c.num_classes, c.transform,
                            c.initial_value, c.num_features)
    finally:
        _rt.TB_FreeForest(h)


def GenerateLLVMIRForXGBoostModel(modelJSONPathStr, llvmIRPathStr, modelGlobalsJSONPathStr, options):
    _rt.GenerateLLVMIRForXGBoostModel(modelJSONPathStr.encode("ascii"), llvmIRPathStr.encode("ascii"),
                                      modelGlobalsJSONPathStr.encode("ascii"), options.optionsPtr)
    treebeardAPI.check()


def SetDevices(devices):
    """CUDA devices of the runners built from now on (no counterpart in the reference): one
    device id, or several -- a runner then keeps the forest on each of them and splits every
    host batch into one row range per device."""
    devices = [int(d) for d in (devices if hasattr(devices, "__iter__") else [devices])]
    arr = (ctypes.c_int32 * len(devices))(*devices)
    _rt.TB_SetDevices(ctypes.addressof(arr), len(devices))


def SetEnableSparseRepresentation(val):
    _rt.SetEnableSparseRepresentation(1 if val else 0)


def IsSparseRepresentationEnabled():
    return _rt.IsSparseRepresentationEnabled()


def SetPeeledCodeGenForProbabilityBasedTiling(val):
    _rt.SetPeeledCodeGenForProbabilityBasedTiling(1 if val else 0)


def IsPeeledCodeGenForProbabilityBasedTilingEnabled():
    return _rt.IsPeeledCodeGenForProbabilityBasedTilingEnabled()


def SetEnableMeasureGpuKernelTime(val):
    _rt.SetEnableMeasureGpuKernelTime(bool(val))


def SetNumberOfKernelRuns(val):
    _rt.SetNumberOfKernelRuns(val)


def GetGPUKernelExecutionTime(inferenceRunner):
    return _rt.GetGPUKernelExecutionTime(inferenceRunner.inferenceRunner)
