"""ctypes binding table for the inference-runner C API (include/tbruntime.h).

Mirrors the role of the reference's src/python/treebeard_runtime_api.py: one object,
``TreebeardAPI``, whose ``runtime_lib`` attribute is the loaded library with argument
and result types set, plus thin methods for the calls that take strings.  Entry-point
names and signatures are the reference's; handles travel as 64-bit integers."""
import ctypes

from . import _lib

_I64, _I32, _VP, _CP, _B = (ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p, ctypes.c_char_p,
                            ctypes.c_bool)

# name -> (argument types, result type)
_SIGNATURES = {
    "InitializeInferenceRunner": ((_CP, _CP), _I64),
    "RunInference": ((_I64, _VP, _VP), None),
    "RunInferenceOnMultipleBatches": ((_I64, _VP, _VP, _I32), None),
    "GetBatchSize": ((_I64,), _I32),
    "GetRowSize": ((_I64,), _I32),
    "DeleteInferenceRunner": ((_I64,), None),
    "CreateCompilerOptions": ((), _I64),
    "DeleteCompilerOptions": ((_I64,), None),
    "Set_statsProfileCSVPath": ((_I64, _CP), None),
    "CreateGPUAutoScheduleOptions": ((), _I64),
    "DeleteGPUAutoScheduleOptions": ((_I64,), None),
    "GenerateLLVMIRForXGBoostModel": ((_CP, _CP, _CP, _I64), None),
    "CreateInferenceRunner": ((_CP, _CP, _I64), _I64),
    "CreateLLVMIRForONNXModel": ((_CP, _CP, _CP, _I64), None),
    "CreateInferenceRunnerForONNXModel": ((_CP, _I64), _I64),
    "SetEnableSparseRepresentation": ((_I32,), None),
    "IsSparseRepresentationEnabled": ((), _I32),
    "SetPeeledCodeGenForProbabilityBasedTiling": ((_I32,), None),
    "IsPeeledCodeGenForProbabilityBasedTilingEnabled": ((), _I32),
    "SetEnableMeasureGpuKernelTime": ((_B,), None),
    "SetNumberOfKernelRuns": ((_I32,), None),
    "ConstructRepresentation": ((_CP,), _I64),
    "DestroyRepresentation": ((_I64,), None),
    "ConstructTreebeardContext": ((_CP, _CP, _I64), _I64),
    "ConstructTreebeardContextFromGPUAutoscheduleOptions": ((_CP, _CP, _I64, _I64), _I64),
    "DestroyTreebeardContext": ((_I64,), None),
    "SetForestCreatorType": ((_I64, _CP), None),
    "SetRepresentationAndSerializer": ((_I64, _CP), None),
    "GetScheduleFromTBContext": ((_I64,), _I64),
    "BuildHIRRepresentation": ((_I64,), None),
    "LowerToLLVMAndDumpIR": ((_I64, _CP), _B),
    "ConstructInferenceRunnerFromHIR": ((_I64,), _I64),
    "ConstructGPUInferenceRunnerFromHIR": ((_I64,), _I64),
    "ConstructGPUInferenceRunnerFromTBContext": ((_I64,), _I64),
    "findBestGPUScheduleAndCompileModel": ((_I64,), _I64),
    "SetOneTreeAtATimeSchedule": ((_I64,), None),
    "Schedule_NewIndexVariable": ((_I64, _CP), _I64),
    "Schedule_NewIndexVariable2": ((_I64, _I64), _I64),
    "Schedule_Tile": ((_I64, _I64, _I64, _I64, _I32), None),
    "Schedule_Reorder": ((_I64, _VP, _I32), None),
    "Schedule_Split": ((_I64, _I64, _I64, _I64, _I32, _I64), None),
    "Schedule_Specialize": ((_I64, _I64), _I64),
    "GetSpecializationInfoNumIterations": ((_I64,), _I64),
    "GetSpecializationInfoNumEntries": ((_I64,), _I64),
    "GetSpecializationInfoEntries": ((_I64, _VP, _VP), None),
    "Schedule_Pipeline": ((_I64, _I64, _I32), None),
    "Schedule_Simdize": ((_I64, _I64), None),
    "Schedule_Parallel": ((_I64, _I64), None),
    "Schedule_Unroll": ((_I64, _I64), None),
    "Schedule_PeelWalk": ((_I64, _I64, _I32), None),
    "Schedule_Cache": ((_I64, _I64), None),
    "Schedule_GetRootIndex": ((_I64,), _I64),
    "Schedule_GetBatchIndex": ((_I64,), _I64),
    "Schedule_GetTreeIndex": ((_I64,), _I64),
    "Schedule_PrintToString": ((_I64, _VP, _I32), _I32),
    "Schedule_GetBatchSize": ((_I64,), _I32),
    "Schedule_GetForestSize": ((_I64,), _I32),
    "Schedule_IsDefaultSchedule": ((_I64,), _B),
    "Schedule_Finalize": ((_I64,), None),
    "Schedule_AtomicReduce": ((_I64, _I64), None),
    "Schedule_VectorReduce": ((_I64, _I64, _I32), None),
    "Schedule_SharedReduce": ((_I64, _I64), None),
    "IndexVariable_SetGPUThreadDim": ((_I64, _I32, _I32), None),
    "GetGPUKernelExecutionTime": ((_I64,), _I64),
    "TB_GetLastStatus": ((), _I32),
    "TB_GetLastError": ((), _CP),
    "TB_SetDevice": ((_I32,), None),
    "TB_SetDevices": ((_VP, _I32), None),
    "TB_RunnerDeviceCount": ((_I64,), _I32),
    "TB_GetKernelForest": ((_I64,), _I64),
    "TB_CreateInferenceRunnerFromArrays": ((_VP, _I64, _I64, _CP), _I64),
    "TB_LoadForest": ((_CP, _CP, _I32), _I64),
    "TB_ForestGetArrays": ((_I64, _VP), _I32),
    "TB_FreeForest": ((_I64,), None),
    "TB_RunnerUsedPackedImage": ((_I64,), _I32),
    "TB_GetInputTypeBitWidth": ((_I64,), _I32),
    "TB_GetReturnTypeBitWidth": ((_I64,), _I32),
}
for _name in ("numberOfFeatures", "batchSize", "tileSize", "thresholdTypeWidth", "returnTypeWidth",
              "returnTypeFloatType", "featureIndexTypeWidth", "nodeIndexTypeWidth",
              "inputElementTypeWidth", "tileShapeBitWidth", "childIndexBitWidth",
              "makeAllLeavesSameDepth", "reorderTreesByDepth", "pipelineSize", "numberOfCores",
              "numParallelTreeBatches", "tilingType", "numRowsPerTB", "numRowsPerThread",
              "rowTileSize", "numTreeThreads", "numTreesAtATime", "cacheRows", "cacheTrees",
              "unrollTreeWalks", "treeWalkInterleaveFactor", "sharedMemoryReduce"):
    _SIGNATURES["Set_" + _name] = ((_I64, _I32), None)

EXPORTED_NAMES = tuple(sorted(_SIGNATURES))


class TreebeardRuntimeError(RuntimeError):
    pass


class TreebeardAPI:
    def __init__(self) -> None:
        self.runtime_lib = _lib.load()
        for name, (args, res) in _SIGNATURES.items():
            fn = getattr(self.runtime_lib, name)
            fn.argtypes = list(args)
            fn.restype = res

    # the reference aborts on errors; here every wrapper call can be followed by check()
    def check(self):
        status = self.runtime_lib.TB_GetLastStatus()
        if status != 0:
            raise TreebeardRuntimeError(
                f"status {status}: {self.runtime_lib.TB_GetLastError().decode()}")

    @staticmethod
    def _s(text):
        return text.encode("ascii") if isinstance(text, str) else text

    def InitializeInferenceRunner(self, soPath, globalsPath):
        return self.runtime_lib.InitializeInferenceRunner(self._s(soPath), self._s(globalsPath))

    def RunInference(self, runner, inputs, results):
        self.runtime_lib.RunInference(runner, inputs, results)
        self.check()

    def RunInferenceOnMultipleBatches(self, runner, inputs, results, numRows):
        self.runtime_lib.RunInferenceOnMultipleBatches(runner, inputs, results, numRows)
        self.check()

    def GetBatchSize(self, runner):
        return self.runtime_lib.GetBatchSize(runner)

    def GetRowSize(self, runner):
        return self.runtime_lib.GetRowSize(runner)

    def DeleteInferenceRunner(self, runner):
        self.runtime_lib.DeleteInferenceRunner(runner)

    def ConstructTreebeardContext(self, modelPath, globalsPath, options):
        return self.runtime_lib.ConstructTreebeardContext(self._s(modelPath), self._s(globalsPath),
                                                          options)

    def ConstructTreebeardContextFromGPUAutoscheduleOptions(self, modelPath, globalsPath, options,
                                                            gpuOptions):
        return self.runtime_lib.ConstructTreebeardContextFromGPUAutoscheduleOptions(
            self._s(modelPath), self._s(globalsPath), options, gpuOptions)

    def DestroyTreebeardContext(self, ctx):
        self.runtime_lib.DestroyTreebeardContext(ctx)

    def SetForestCreatorType(self, ctx, name):
        self.runtime_lib.SetForestCreatorType(ctx, self._s(name))
        self.check()

    def SetRepresentationAndSerializer(self, ctx, name):
        self.runtime_lib.SetRepresentationAndSerializer(ctx, self._s(name))
        self.check()

    def GetScheduleFromTBContext(self, ctx):
        return self.runtime_lib.GetScheduleFromTBContext(ctx)

    def LowerToLLVMAndDumpIR(self, ctx, path):
        return self.runtime_lib.LowerToLLVMAndDumpIR(ctx, self._s(path))

    def __getattr__(self, name):
        # Schedule_* and the remaining plain entry points pass straight through
        if name in _SIGNATURES:
            fn = getattr(self.runtime_lib, name)
            if _CP in _SIGNATURES[name][0]:
                return lambda *a: fn(*[self._s(x) for x in a])
            return fn
        raise AttributeError(name)
