"""Host-side behaviour of the inference-runner API that needs no GPU: options, contexts,
model loading, schedule objects, error reporting, launch-shape selection."""
import os

import numpy as np
import pytest

from tests.helpers import small_config
from treebeard_b200 import kernels, synth, treebeard


def test_context_loads_model_and_reports_schedule(tmp_path):
    forest, _ = small_config("c1", rows=1)
    path = str(tmp_path / "c1.json")
    synth.save_xgboost_json(forest, path)
    options = treebeard.CompilerOptions(512, 1)
    ctx = treebeard.TreebeardContext(path, "", options)
    ctx.SetInputFiletype("xgboost_json")
    ctx.SetRepresentationType("gpu_sparse")
    ctx.BuildHIRRepresentation()
    sched = ctx.GetSchedule()
    assert sched.GetBatchSize() == 512 and sched.GetForestSize() == 100
    assert sched.IsDefaultSchedule()
    batch, tree = sched.GetBatchIndex(), sched.GetTreeIndex()
    b0, b1 = sched.NewIndexVariable("b0"), sched.NewIndexVariable("b1")
    sched.Tile(batch, b0, b1, 32)
    sched.Reorder([b0, tree, b1])
    b0.set_gpu_dimension(treebeard.GPUConstruct.Grid, treebeard.Dimension.X)
    sched.Cache(b0)
    sched.SharedReduce(tree)
    text = sched.PrintToString()
    assert "tile(batch -> b0, b1, 32)" in text and "reorder(b0, tree, b1)" in text
    assert not sched.IsDefaultSchedule()


def test_bad_inputs_report_errors_instead_of_aborting(tmp_path):
    options = treebeard.CompilerOptions(64, 1)
    ctx = treebeard.TreebeardContext(str(tmp_path / "missing.json"), "", options)
    with pytest.raises(treebeard.TreebeardRuntimeError):
        ctx.SetInputFiletype("lightgbm_txt")
    with pytest.raises(treebeard.TreebeardRuntimeError):
        ctx.SetRepresentationType("gpu_fancy")
    ctx.SetInputFiletype("xgboost_json")
    with pytest.raises(treebeard.TreebeardRuntimeError, match="cannot open"):
        ctx.BuildHIRRepresentation()
    bad = tmp_path / "bad.json"
    bad.write_text('{"learner": {"learner_model_param": {"base_score": "0.5"}')
    ctx2 = treebeard.TreebeardContext(str(bad), "", options)
    with pytest.raises(treebeard.TreebeardRuntimeError, match="JSON"):
        ctx2.BuildHIRRepresentation()
    # dumping a model that cannot be read fails on the model, and writes nothing
    with pytest.raises(treebeard.TreebeardRuntimeError, match="cannot open"):
        ctx.DumpLLVMIR(str(tmp_path / "x.tbmodel"))
    assert not (tmp_path / "x.tbmodel").exists()


def test_unknown_objective_is_an_error(tmp_path):
    forest, _ = small_config("c1", rows=1)
    model = synth.to_xgboost_dict(forest)
    model["learner"]["objective"]["name"] = "rank:pairwise"
    import json
    path = tmp_path / "m.json"
    path.write_text(json.dumps(model))
    ctx = treebeard.TreebeardContext(str(path), "", treebeard.CompilerOptions(64, 1))
    with pytest.raises(treebeard.TreebeardRuntimeError, match="objective"):
        ctx.BuildHIRRepresentation()


def test_global_switches_round_trip():
    treebeard.SetEnableSparseRepresentation(True)
    assert treebeard.IsSparseRepresentationEnabled() == 1
    treebeard.SetEnableSparseRepresentation(False)
    assert treebeard.IsSparseRepresentationEnabled() == 0
    treebeard.SetPeeledCodeGenForProbabilityBasedTiling(True)
    assert treebeard.IsPeeledCodeGenForProbabilityBasedTilingEnabled() == 1
    treebeard.SetPeeledCodeGenForProbabilityBasedTiling(False)


CASES = {  # name: (F, classes, trees, largest group bytes, rows)
    "c1": (8, 0, 100, 16256, 1024), "c2": (28, 0, 1000, 50000, 1048576),
    "c2_small": (28, 0, 1000, 50000, 4096), "c3": (2000, 0, 1000, 65408, 262144),
    "c4": (16, 26, 2600, 56192, 1048576), "c5": (128, 0, 16000, 1048448, 4194304)}


@pytest.mark.parametrize("name", list(CASES))
def test_launch_plans_fit_the_device(name):
    F, C, T, gbytes, rows = CASES[name]
    info = kernels.plan_launch(F, C, (T + 15) // 16, gbytes, rows)
    s = info.schedule
    assert info.smem_bytes <= 232448
    assert 32 <= info.threads_per_block <= 1024 and info.threads_per_block % 32 == 0
    assert s.tree_threads in (1, 2, 4, 8, 16)
    assert s.rows_per_block % 32 == 0 and s.rows_per_block >= 32
    grid_x = info.reserved[1]
    assert grid_x * s.rows_per_block >= rows
    assert s.tree_chunks * info.reserved[2] >= (T + 15) // 16
    if name == "c5":
        assert info.staged == 0       # a 1 MB tree group cannot be staged
    if name in ("c1", "c2", "c4"):
        assert info.staged == 1 and info.reserved[0] == 1
    if name in ("c1", "c2_small"):
        # small batches still fill the GPU, as far as the number of tree groups allows
        assert grid_x * s.tree_chunks >= min(148, grid_x * ((T + 15) // 16))


def test_launch_plan_honours_user_schedule():
    info = kernels.plan_launch(28, 0, 63, 50000, 65536, rows_per_block=64, tree_threads=4,
                               tree_chunks=3, rows_per_thread=2)
    assert info.schedule.rows_per_block == 64 and info.schedule.tree_threads == 4
    assert info.schedule.tree_chunks == 3 and info.schedule.rows_per_thread == 2
    with pytest.raises(kernels.TbkError):
        kernels.plan_launch(128, 0, 1000, 1048448, 4096, cache_trees=1)


@pytest.mark.parametrize("classes", [2, 3, 6, 26])
def test_partial_sum_plans_always_hold_the_class_table(classes):
    """A launch that writes per-class partial sums (tree shards, the entry point that does not
    allocate) sums classes through a per-warp table in shared memory.  At large batches the
    selector keeps class sums in registers and drops that table -- but never for such a launch:
    its shared-memory size must include warps x classes x 32 floats."""
    F, groups, gbytes = 28, 20, 20000
    rows = 400000                                     # > 2 x 148 SMs x 32 warps x 32 rows
    direct = kernels.plan_launch(F, classes, groups, gbytes, rows)
    assert direct.reserved[3] == 1                    # predictions: class sums in registers
    part = kernels.plan_launch(F, classes, groups, gbytes, rows, partial_sums=True)
    assert part.reserved[3] == 0
    warps = part.threads_per_block // 32
    rt = 32 * part.schedule.rows_per_thread
    table = warps * classes * rt * 4
    rows_cache = (part.schedule.rows_per_block // rt) * (F + 1) * rt * 4
    assert part.smem_bytes >= table + rows_cache
    assert part.smem_bytes <= 232448
