"""The C-ABI library loads without a GPU and exports every symbol the headers declare."""
import ctypes
import os
import re

import pytest

from treebeard_b200 import _lib, treebeard_runtime_api

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared(header, macro):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("#"))
    names = []
    for m in re.finditer(macro + r"\s+([^;{]*?)\(", text):
        names.append(m.group(1).split()[-1].lstrip("*"))
    return names


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    tbk = declared("tbk.h", "TBK_EXPORT")
    rt = declared("tbruntime.h", "TREEBEARD_RUNTIME_EXPORT")
    assert len(tbk) >= 15 and len(rt) >= 90
    for name in tbk + rt:
        assert hasattr(lib, name), f"{name} is declared but not exported"


def test_binding_table_covers_the_runtime_header():
    rt = set(declared("tbruntime.h", "TREEBEARD_RUNTIME_EXPORT"))
    assert rt == set(treebeard_runtime_api.EXPORTED_NAMES)


def test_reference_entry_points_are_present():
    # the names the reference's ctypes table binds (src/python/treebeard_runtime_api.py)
    lib = _lib.load()
    for name in ("RunInference", "RunInferenceOnMultipleBatches", "GetBatchSize", "GetRowSize",
                 "DeleteInferenceRunner", "CreateCompilerOptions", "CreateGPUAutoScheduleOptions",
                 "ConstructTreebeardContext", "ConstructTreebeardContextFromGPUAutoscheduleOptions",
                 "SetForestCreatorType", "SetRepresentationAndSerializer",
                 "ConstructGPUInferenceRunnerFromTBContext", "findBestGPUScheduleAndCompileModel",
                 "GetGPUKernelExecutionTime", "SetEnableMeasureGpuKernelTime", "Schedule_Tile"):
        assert isinstance(getattr(lib, name), ctypes._CFuncPtr)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(ImportError, match="no fallback"):
        _lib.load()
