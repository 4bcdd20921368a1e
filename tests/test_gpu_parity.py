"""GPU parity tests: the CUDA path, called through the C ABI, against the CPU oracle.

Bars: the selected leaf per (row, tree) is bit-exact; fp32 predictions are within
1e-5 relative / 1e-6 absolute of the oracle (summation order differs); class ids are
exact except where the two best class sums tie within rounding."""
import os

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import (SMALL, assert_predictions_close, golden_forest, small_config)

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _dev(x):
    return torch.from_numpy(np.ascontiguousarray(x)).cuda()


REPS = [("sparse", 1), ("array", 1), ("reorg", 1), ("sparse", 2), ("sparse", 3), ("sparse", 4),
        ("array", 3), ("array", 4)]


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("rep,ts", REPS)
def test_config_parity(name, rep, ts):
    from treebeard_b200 import kernels
    if name == "c5" and rep == "array" and ts > 1:
        pytest.skip("array layout of deep unbalanced trees is too large by construction")
    forest, X = small_config(name)
    want, want_ids, sums = oracle.predict(forest, X, leaf_ids=True, class_sums=True)
    df = kernels.DeviceForest(forest, representation=rep, tile_size=ts, batch_hint=len(X))
    dX = _dev(X)
    ids = df.predict_leaf_ids(dX).cpu().numpy()
    assert np.array_equal(ids, want_ids), f"{(ids != want_ids).sum()} leaf ids differ"
    got = df.predict(dX).cpu().numpy()
    df.check_status()
    assert_predictions_close(got, want, forest, sums)
    if forest.num_classes > 0:
        got8 = df.predict(dX, int8=True).cpu().numpy()
        assert np.array_equal(got8.astype(np.float32), got)


@pytest.mark.parametrize("name", ["c2", "c4", "c5"])
@pytest.mark.parametrize("sched", [dict(tree_threads=4), dict(tree_chunks=3), dict(rows_per_thread=2),
                                   dict(tree_threads=16, tree_chunks=2), dict(cache_trees=2),
                                   dict(rows_per_block=64, tree_threads=2)])
def test_schedule_variants(name, sched):
    from treebeard_b200 import kernels
    forest, X = small_config(name)
    want, sums = oracle.predict(forest, X, class_sums=True)
    df = kernels.DeviceForest(forest, representation="sparse", batch_hint=len(X), **sched)
    got = df.predict(_dev(X)).cpu().numpy()
    df.check_status()
    assert_predictions_close(got, want, forest, sums)


@pytest.mark.parametrize("n", [1, 31, 33, 100, 1025])
def test_ragged_batches_and_strides(n):
    from treebeard_b200 import kernels
    forest, X = small_config("c2", rows=n)
    want = oracle.predict(forest, X)
    df = kernels.DeviceForest(forest, representation="sparse")
    # padded row stride that breaks 16-byte alignment of rows: the scalar staging path
    wide = torch.zeros((n, forest.num_features + 3), device="cuda")
    wide[:, :forest.num_features] = _dev(X)
    got = df.predict(wide[:, :forest.num_features]).cpu().numpy()
    assert_predictions_close(got, want)
    got2 = df.predict(_dev(X)).cpu().numpy()
    assert_predictions_close(got2, want)


def test_empty_batch_and_errors():
    from treebeard_b200 import kernels
    forest, X = small_config("c1", rows=8)
    df = kernels.DeviceForest(forest)
    out = df.predict(torch.empty((0, forest.num_features), device="cuda"))
    assert out.numel() == 0
    with pytest.raises(kernels.TbkError):
        df.predict(_dev(X), int8=True)  # int8 output needs a multiclass forest


def test_nan_and_ties_go_right():
    from treebeard_b200 import kernels
    forest, X = small_config("c4", rows=512)  # integer features: x == threshold is common
    X = X.copy()
    X[::7, ::3] = np.nan
    X[::11, 1] = np.inf
    X[::13, 2] = -np.inf
    want, want_ids = oracle.predict(forest, X, leaf_ids=True)
    df = kernels.DeviceForest(forest)
    ids = df.predict_leaf_ids(_dev(X)).cpu().numpy()
    assert np.array_equal(ids, want_ids)


def test_partial_and_finalize_match_predict():
    from treebeard_b200 import kernels
    for name in ("c2", "c4"):
        forest, X = small_config(name)
        want, sums = oracle.predict(forest, X, class_sums=True)
        half = forest.num_trees // 2
        a = kernels.DeviceForest(forest.tree_slice(0, half))
        b = kernels.DeviceForest(forest.tree_slice(half, forest.num_trees), tree_chunks=2)
        dX = _dev(X)
        total = a.predict_partial(dX) + b.predict_partial(dX)
        got = a.finalize(total).cpu().numpy()
        assert_predictions_close(got, want, forest, sums)


def test_host_pipeline_matches_device_path():
    from treebeard_b200 import kernels
    forest, X = small_config("c2", rows=70000)
    df = kernels.DeviceForest(forest)
    dev = df.predict(_dev(X)).cpu().numpy()
    host = df.predict_host(X)
    assert np.array_equal(dev, host)
    pinned = torch.from_numpy(X).pin_memory()
    out = torch.empty(len(X), dtype=torch.float32).pin_memory()
    df.predict_host(pinned.numpy(), out.numpy())
    assert np.array_equal(out.numpy(), dev)


@pytest.mark.parametrize("model", ["higgs", "airline", "year_prediction_msd"])
def test_golden_benchmark_models(model, golden_dir):
    from treebeard_b200 import kernels
    z = np.load(os.path.join(golden_dir, model + ".npz"))
    forest = golden_forest(z)
    for rep in ("sparse", "array", "reorg"):
        df = kernels.DeviceForest(forest, representation=rep)
        got = df.predict(_dev(z["rows"])).cpu().numpy()
        # the reference's own tolerance against XGBoost's predictions
        assert oracle.fp_equal(got, z["expected"]).all()
        assert_predictions_close(got, oracle.predict(forest, z["rows"]))


@pytest.mark.parametrize("stem", ["TestModel_Size1_1", "TestModel_Size1_8", "TestModel_Size2_1",
                                  "TestModel_Size2_13", "TestModel_Size4_1", "TestModel_Size4_10",
                                  "leftheavy_xgb_model", "rightheavy_xgb_model",
                                  "rightandleftheavy_xgb_model"])
@pytest.mark.parametrize("rep", ["gpu_sparse", "gpu_array", "gpu_reorg"])
def test_runner_api_on_golden_json(stem, rep, golden_dir):
    """The reference-shaped flow: options -> context -> representation -> GPU runner."""
    from treebeard_b200 import treebeard
    z = np.load(os.path.join(golden_dir, stem + ".npz"))
    rows, expected = z["rows"], z["expected"]
    batch = 64
    options = treebeard.CompilerOptions(batch, 1)
    ctx = treebeard.TreebeardContext(os.path.join(golden_dir, stem + ".json"), "", options)
    ctx.SetInputFiletype("xgboost_json")
    ctx.SetRepresentationType(rep)
    runner = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    assert runner.batchSize == batch and runner.rowSize == rows.shape[1]
    got = runner.RunInference(np.ascontiguousarray(rows[:batch]))
    assert oracle.fp_equal(got, expected[:batch]).all()
    many = runner.RunInferenceOnMultipleBatches(np.ascontiguousarray(rows[:4 * batch]))
    assert oracle.fp_equal(many, expected[:4 * batch]).all()
    on_dev = runner.RunInference(_dev(rows[:batch])).cpu().numpy()
    assert np.array_equal(on_dev, got)


def test_runner_without_a_named_representation_gets_the_librarys_choice(golden_dir):
    """No SetRepresentationType and the process-wide sparse switch untouched: "gpu_auto", which
    lays this single-output forest out as keys; same predictions as the named layouts."""
    from treebeard_b200 import kernels, treebeard
    if treebeard.IsSparseRepresentationEnabled():
        pytest.skip("the process-wide sparse switch is set")
    z = np.load(os.path.join(golden_dir, "TestModel_Size2_13.npz"))
    rows, expected = z["rows"], z["expected"]
    options = treebeard.CompilerOptions(64, 1)
    ctx = treebeard.TreebeardContext(os.path.join(golden_dir, "TestModel_Size2_13.json"), "", options)
    ctx.SetInputFiletype("xgboost_json")
    runner = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    got = runner.RunInference(np.ascontiguousarray(rows[:64]))
    assert oracle.fp_equal(got, expected[:64]).all()
    handle = runner.kernel_forest()
    if handle:
        df = kernels.DeviceForest.from_handle(handle, 0, 1, 0, rows.shape[1])
        assert df.info().schedule.feature_bits in (16, 32)   # 16 unless an earlier test set the switch


def test_runner_over_several_devices(tmp_path):
    """One runner, a copy of the forest per device, host batches cut into one row range per
    device and predicted concurrently (here the same device named twice, or two devices where
    the box has them)."""
    from treebeard_b200 import synth, treebeard
    forest, X = small_config("c2", rows=17 * 256)
    path = str(tmp_path / "c2.json")
    synth.save_xgboost_json(forest, path)
    want = oracle.predict(forest, X)
    second = 1 if torch.cuda.device_count() > 1 else 0
    treebeard.SetDevices([0, second])
    try:
        options = treebeard.CompilerOptions(256, 1)
        ctx = treebeard.TreebeardContext(path, "", options)
        ctx.SetRepresentationType("gpu_auto")
        runner = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    finally:
        treebeard.SetDevices([0])
    assert runner.device_count() == 2
    assert_predictions_close(runner.RunInferenceOnMultipleBatches(X), want)
    assert_predictions_close(runner.RunInference(np.ascontiguousarray(X[:256])), want[:256])
    single = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    assert single.device_count() == 1


def test_runner_with_64_bit_types(golden_dir):
    """The reference's other tested type combination (f64 thresholds and values, i32 indices,
    src/test/GPUTests.cpp:682-840): host buffers hold doubles, the walk computes in fp32."""
    from treebeard_b200 import treebeard
    z = np.load(os.path.join(golden_dir, "TestModel_Size2_13.npz"))
    rows, expected = z["rows"], z["expected"]
    batch = 64
    options = treebeard.CompilerOptions(batch, 1)
    options.SetThresholdTypeWidth(64)
    options.SetInputElementTypeWidth(64)
    options.SetReturnTypeWidth(64)
    options.SetFeatureIndexTypeWidth(32)
    options.SetNodeIndexTypeWidth(32)
    ctx = treebeard.TreebeardContext(os.path.join(golden_dir, "TestModel_Size2_13.json"), "", options)
    ctx.SetInputFiletype("xgboost_json")
    ctx.SetRepresentationType("gpu_sparse")
    runner = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    wide = np.ascontiguousarray(rows[:4 * batch], np.float64)
    got = runner.RunInference(wide[:batch], np.float64)
    assert got.dtype == np.float64 and oracle.fp_equal(got, expected[:batch]).all()
    many = runner.RunInferenceOnMultipleBatches(wide, np.float64)
    assert oracle.fp_equal(many, expected[:4 * batch]).all()
    with pytest.raises(treebeard.TreebeardRuntimeError):
        runner.RunInference(wide[:batch])                    # the runner returns float64
    with pytest.raises(treebeard.TreebeardRuntimeError, match="host"):
        dev = torch.zeros((batch, rows.shape[1]), device="cuda")
        out = torch.zeros(batch, device="cuda")
        runner.treebeardAPI.RunInference(runner.inferenceRunner, dev.data_ptr(), out.data_ptr())


def test_runner_multiclass_int8(tmp_path):
    from treebeard_b200 import synth, treebeard
    forest, X = small_config("c4", rows=256)
    path = str(tmp_path / "c4.json")
    synth.save_xgboost_json(forest, path)
    want, sums = oracle.predict(forest, X, class_sums=True)
    options = treebeard.CompilerOptions(256, 1)
    options.SetReturnTypeWidth(8)
    options.SetReturnTypeIsFloatType(False)
    ctx = treebeard.TreebeardContext(path, "", options,
                                     treebeard.GPUAutoScheduleOptions.Construct(64, 1, 4))
    ctx.SetRepresentationType("gpu_sparse")
    runner = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    got = runner.RunInference(X, np.int8)
    assert_predictions_close(got.astype(np.float32), want, forest, sums)


def test_kernel_timing_api(tmp_path):
    from treebeard_b200 import synth, treebeard
    forest, X = small_config("c1")
    path = str(tmp_path / "c1.json")
    synth.save_xgboost_json(forest, path)
    treebeard.SetEnableMeasureGpuKernelTime(True)
    treebeard.SetNumberOfKernelRuns(3)
    try:
        options = treebeard.CompilerOptions(1024, 1)
        ctx = treebeard.TreebeardContext(path, "", options)
        ctx.SetRepresentationType("gpu_array")
        runner = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
        got = runner.RunInference(X)
        assert treebeard.GetGPUKernelExecutionTime(runner) > 0
        assert_predictions_close(got, oracle.predict(forest, X))
    finally:
        treebeard.SetEnableMeasureGpuKernelTime(False)
        treebeard.SetNumberOfKernelRuns(1)


@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_sixteen_bit_key_kernel_is_exact(name):
    """The wide-row kernel (rows staged as 16-bit keys) must select exactly the oracle's
    leaves, ties, NaN and infinities included."""
    from treebeard_b200 import kernels
    forest, X = small_config(name)
    X = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(600):
        g = split[(i * 37) % len(split)]
        X[i % len(X), forest.feat[g]] = forest.thr[g]
    X[3, :] = np.nan
    X[4, 0] = np.inf
    X[5, 1] = -np.inf
    want, want_ids = oracle.predict(forest, X, leaf_ids=True)
    df = kernels.DeviceForest(forest, representation="reorg", feature_bits=16, batch_hint=len(X))
    info = df.info()
    # wide rows: one key tile per block (24 warps); narrow rows: batches of tiles (20 warps)
    assert info.schedule.feature_bits == 16 and info.threads_per_block == (768 if name == "c3" else 704)
    dX = _dev(X)
    ids = df.predict_leaf_ids(dX).cpu().numpy()
    df.check_status()
    assert np.array_equal(ids, want_ids), f"{(ids != want_ids).sum()} leaf ids differ"
    got = df.predict(dX).cpu().numpy()
    df.check_status()
    ok = ~np.isnan(want)
    assert_predictions_close(got[ok], want[ok])
    assert df.info().reserved[0] > 0          # key ties were hit and resolved exactly
    # partial sums + second pass, ragged batch, unaligned rows
    part = df.predict_partial(dX[:777])
    again = df.finalize(part).cpu().numpy()
    assert_predictions_close(again[ok[:777]], want[:777][ok[:777]])
    wide = torch.zeros((len(X), forest.num_features + 1), device="cuda")
    wide[:, :forest.num_features] = dX
    got2 = df.predict(wide[:, :forest.num_features]).cpu().numpy()
    assert np.array_equal(got2[ok], got[ok])


def test_auto_representation_picks_keys_for_single_output_forests_of_up_to_eight_levels():
    """"auto": keys for wide rows (one tile per block) and for narrow rows (batches of tiles,
    multiclass forests included); fp32 tiles on request and for explicit representations."""
    from treebeard_b200 import kernels
    wide, Xw = small_config("c3", rows=64)
    narrow, Xn = small_config("c2", rows=64)
    multi, Xm = small_config("c4", rows=64)
    a = kernels.DeviceForest(wide, representation="auto")
    b = kernels.DeviceForest(narrow, representation="auto")
    assert a.info().schedule.feature_bits == 16 and a.info().threads_per_block == 768
    assert b.info().schedule.feature_bits == 16 and b.info().threads_per_block == 704
    assert kernels.DeviceForest(narrow, representation="auto", feature_bits=32).info().schedule.feature_bits == 32
    assert kernels.DeviceForest(narrow, representation="sparse").info().schedule.feature_bits == 32
    m = kernels.DeviceForest(multi, representation="auto")
    assert m.info().schedule.feature_bits == 16 and m.info().threads_per_block == 704
    assert kernels.DeviceForest(multi, representation="sparse").info().schedule.feature_bits == 32
    want_m, sums_m = oracle.predict(multi, Xm, class_sums=True)
    assert_predictions_close(m.predict(_dev(Xm)).cpu().numpy(), want_m, multi, sums_m)
    assert_predictions_close(a.predict(_dev(Xw)).cpu().numpy(), oracle.predict(wide, Xw))
    assert_predictions_close(b.predict(_dev(Xn)).cpu().numpy(), oracle.predict(narrow, Xn))
    # whole-number thresholds (integer-valued features: rows EQUAL thresholds all the time) become
    # lattice features of the key layout: exact without a single tie on whole-number rows
    import copy
    rounded = copy.copy(narrow)
    rounded.thr = np.where(narrow.left >= 0, np.round(narrow.thr * 4), narrow.thr).astype(np.float32)
    Xr = np.round(Xn * 4).astype(np.float32)
    c = kernels.DeviceForest(rounded, representation="auto")
    assert c.info().schedule.feature_bits == 16
    want, want_ids = oracle.predict(rounded, Xr, leaf_ids=True)
    assert np.array_equal(c.predict_leaf_ids(_dev(Xr)).cpu().numpy(), want_ids)
    assert_predictions_close(c.predict(_dev(Xr)).cpu().numpy(), want)
    assert c.info().reserved[0] == 0


@pytest.mark.parametrize("name,rows,chunks", [("c2", 100003, 0), ("c2", 100003, 3), ("c1", 77777, 0), ("c2", 5000, 0)])
def test_batched_key_kernel_is_exact(name, rows, chunks):
    """Narrow rows: the key tiles of up to 16 tiles are staged together and the forest streams
    once per batch.  Full batches, persistent blocks with several batches, a ragged last
    batch and tile, tree chunks, partial sums and leaf ids; ties, NaN and infinities included."""
    from treebeard_b200 import kernels
    forest, X = small_config(name, rows=rows)
    X = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(3000):
        g = split[(i * 37) % len(split)]
        X[(i * 31) % len(X), forest.feat[g]] = forest.thr[g]
    X[3, :] = np.nan
    X[rows - 1, 0] = np.inf
    X[rows // 2, 1] = -np.inf
    want, want_ids = oracle.predict(forest, X, leaf_ids=True)
    df = kernels.DeviceForest(forest, representation="auto", batch_hint=rows, tree_chunks=chunks)
    info = df.info()
    assert info.schedule.feature_bits == 16 and info.threads_per_block == 704
    dX = _dev(X)
    got = df.predict(dX).cpu().numpy()
    df.check_status()
    ok = ~np.isnan(want)
    assert_predictions_close(got[ok], want[ok])
    assert df.info().reserved[0] > 0          # key ties were hit and resolved exactly
    sub = slice(rows - 20001, rows) if rows > 20001 else slice(0, rows)
    ids = df.predict_leaf_ids(dX[sub]).cpu().numpy()
    df.check_status()
    assert np.array_equal(ids, want_ids[sub]), f"{(ids != want_ids[sub]).sum()} leaf ids differ"
    part = df.predict_partial(dX[:rows - 13])
    again = df.finalize(part).cpu().numpy()
    assert_predictions_close(again[ok[:rows - 13]], want[:rows - 13][ok[:rows - 13]])


def test_deep_tree_kernel_with_whole_number_thresholds():
    """Integer-valued features on deep trees: lattice features, exact without a tie on
    whole-number rows; rows that are not whole numbers still select the oracle's leaves."""
    import copy
    from treebeard_b200 import kernels
    forest, X = small_config("c5", rows=3000, trees=12)
    rounded = copy.copy(forest)
    rounded.thr = np.where(forest.left >= 0, np.round(forest.thr * 8), forest.thr).astype(np.float32)
    Xr = np.round(X * 8).astype(np.float32)
    df = kernels.DeviceForest(rounded, representation="auto", batch_hint=len(Xr))
    assert df.info().schedule.feature_bits == 16
    want, want_ids = oracle.predict(rounded, Xr, leaf_ids=True)
    assert np.array_equal(df.predict_leaf_ids(_dev(Xr)).cpu().numpy(), want_ids)
    assert_predictions_close(df.predict(_dev(Xr)).cpu().numpy(), want)
    assert df.info().reserved[0] == 0
    Y = Xr.copy()
    split = np.nonzero(rounded.left >= 0)[0]
    for i in range(3000):
        g = split[(i * 53) % len(split)]
        Y[i % len(Y), rounded.feat[g]] = rounded.thr[g] + ((-1) ** i) * [1e-5, 1e-2, 0.5][i % 3]
    _, want_ids = oracle.predict(rounded, Y, leaf_ids=True)
    assert np.array_equal(df.predict_leaf_ids(_dev(Y)).cpu().numpy(), want_ids)


@pytest.mark.parametrize("trees,rows", [(1, 70), (24, 1500), (33, 20000)])
def test_deep_tree_kernel_is_exact(trees, rows):
    """Deep trees (12 levels): whole trees staged through shared memory over a tile of
    16-bit keys.  Leaves must be exactly the oracle's, ties, NaN and infinities included;
    covers an odd tree count, ragged tiles, tree chunks and the partial-sum path."""
    from treebeard_b200 import kernels
    forest, X = small_config("c5", rows=rows, trees=trees)
    X = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(600):
        g = split[(i * 101) % len(split)]
        X[i % len(X), forest.feat[g]] = forest.thr[g]
    for i in range(6, 60):
        g = forest.tree_off[i % trees]
        X[i, forest.feat[g]] = forest.thr[g]
    X[3, :] = np.nan
    X[4, 0] = np.inf
    X[5, 1] = -np.inf
    want, want_ids = oracle.predict(forest, X, leaf_ids=True)
    df = kernels.DeviceForest(forest, representation="auto", batch_hint=len(X))
    info = df.info()
    assert info.schedule.feature_bits == 16 and info.num_groups == (trees + 1) // 2
    dX = _dev(X)
    ids = df.predict_leaf_ids(dX).cpu().numpy()
    df.check_status()
    assert np.array_equal(ids, want_ids), f"{(ids != want_ids).sum()} leaf ids differ"
    got = df.predict(dX).cpu().numpy()
    df.check_status()
    ok = ~np.isnan(want)
    assert_predictions_close(got[ok], want[ok])
    assert df.info().reserved[0] > 0          # key ties were hit and resolved exactly
    n = min(777, rows)
    part = df.predict_partial(dX[:n])
    again = df.finalize(part).cpu().numpy()
    assert_predictions_close(again[ok[:n]], want[:n][ok[:n]])
    # explicit tree chunks and a padded row stride
    chunked = kernels.DeviceForest(forest, representation="auto", tree_chunks=3, batch_hint=len(X))
    wide = torch.zeros((len(X), forest.num_features + 3), device="cuda")
    wide[:, :forest.num_features] = dX
    got2 = chunked.predict(wide[:, :forest.num_features]).cpu().numpy()
    chunked.check_status()
    assert_predictions_close(got2[ok], want[ok])
    # the fp32 global-memory walk of the same forest agrees
    plain = kernels.DeviceForest(forest, representation="sparse", batch_hint=len(X))
    assert plain.info().schedule.feature_bits == 32
    assert_predictions_close(plain.predict(dX).cpu().numpy()[ok], want[ok])


@pytest.mark.parametrize("mode", ["BRANCH_LT", "BRANCH_GEQ"])
def test_runner_from_onnx_file(mode, tmp_path):
    from treebeard_b200 import synth, treebeard
    forest, X = small_config("c2", rows=512, trees=64)
    path = str(tmp_path / "m.onnx")
    synth.save_onnx(forest, path, mode=mode)
    options = treebeard.CompilerOptions(512, 1)
    options.SetNumberOfFeatures(forest.num_features)
    runner = treebeard.TreebeardInferenceRunner.FromONNXModelFile(path, options)
    assert runner.rowSize == forest.num_features
    assert_predictions_close(runner.RunInference(X), oracle.predict(forest, X))
    ctx = treebeard.TreebeardContext(path, "", options)
    ctx.SetInputFiletype("onnx_file")
    ctx.SetRepresentationType("gpu_sparse")
    again = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx)
    assert_predictions_close(again.RunInference(X), oracle.predict(forest, X))


def test_abalone_onnx_golden_on_gpu(golden_dir):
    from treebeard_b200 import kernels
    z = np.load(os.path.join(golden_dir, "abalone_onnx.npz"))
    forest = golden_forest(z)
    for rep in ("sparse", "array", "reorg"):
        got = kernels.DeviceForest(forest, representation=rep).predict(_dev(z["rows"])).cpu().numpy()
        assert oracle.fp_equal(got, z["expected"]).all()


def test_multiclass_register_class_sums_match_the_class_table_path():
    """Large multiclass batches keep the class sums in registers (class-major groups,
    arg-max decided on the fly); smaller ones and chunked launches use the shared-memory
    class table.  Both must give the oracle's class ids."""
    from treebeard_b200 import kernels, synth
    forest, marg, _ = synth.make_config("c4", trees=78)
    rows = 2 * 148 * 32 * 32 + 77                     # enough row tiles for the register path
    X = synth.config_rows("c4", marg, rows)
    dX = _dev(X)
    fast = kernels.DeviceForest(forest, representation="sparse", batch_hint=rows)
    table = kernels.DeviceForest(forest, representation="sparse", tree_chunks=2, batch_hint=rows)
    a = fast.predict(dX, int8=True).cpu().numpy()
    b = table.predict(dX, int8=True).cpu().numpy()
    fast.check_status()
    assert fast.info().schedule.tree_chunks == 1 and fast.info().threads_per_block == 1024
    pick = np.arange(0, rows, 37)
    want, sums = oracle.predict(forest, X[pick], class_sums=True)
    assert_predictions_close(a[pick], want, forest, sums)
    assert (a != b).mean() < 1e-4                     # only exact class-sum ties may differ
    ids = fast.predict_leaf_ids(dX[:4096]).cpu().numpy()
    _, want_ids = oracle.predict(forest, X[:4096], leaf_ids=True)
    assert np.array_equal(ids, want_ids)


def test_auto_schedule_runner_chooses_the_layout(tmp_path):
    """findBestGPUScheduleAndCompileModel (the reference's timed search over schedules and
    representations) is the layout selector here: deep trees get the deep-tree layout."""
    from treebeard_b200 import kernels, synth, treebeard
    forest, X = small_config("c5", rows=256, trees=6)
    path = str(tmp_path / "deep.json")
    synth.save_xgboost_json(forest, path)
    ctx = treebeard.TreebeardContext(path, "", treebeard.CompilerOptions(256, 1))
    runner = treebeard.TreebeardInferenceRunner.AutoScheduleGPUInferenceRunnerFromTBContext(ctx)
    got = runner.RunInference(X)
    assert_predictions_close(got, oracle.predict(forest, X))
    df = kernels.DeviceForest.from_handle(runner.kernel_forest(), 0, forest.num_trees, 0, forest.num_features)
    assert df.info().schedule.feature_bits == 16
    # an explicit representation keeps its plain meaning
    ctx2 = treebeard.TreebeardContext(path, "", treebeard.CompilerOptions(256, 1))
    ctx2.SetRepresentationType("gpu_sparse")
    plain = treebeard.TreebeardInferenceRunner.GPUInferenceRunnerFromTBContext(ctx2)
    df2 = kernels.DeviceForest.from_handle(plain.kernel_forest(), 0, forest.num_trees, 0, forest.num_features)
    assert df2.info().schedule.feature_bits == 32
    assert_predictions_close(plain.RunInference(X), got)
    # host-resident rows through the chunked pipeline of the kernel library
    out = np.empty(len(X), np.float32)
    df.predict_host(X, out)
    assert_predictions_close(out, got)


@pytest.mark.parametrize("rows", [500, 2 * 148 * 32 * 32])
def test_multiclass_with_an_empty_class(rows):
    """Both multiclass paths (shared-memory class table; class sums in registers) with a
    class that has no trees and strongly negative leaves elsewhere, so that the empty class
    wins on some rows."""
    from treebeard_b200 import kernels, synth
    forest, marg, _ = synth.make_config("c4", trees=52)
    forest.class_id[forest.class_id == 7] = 8
    leaves = forest.left < 0
    forest.thr[leaves] -= np.float32(0.1)              # push every voted class down
    X = synth.config_rows("c4", marg, rows)
    df = kernels.DeviceForest(forest, representation="sparse", batch_hint=rows)
    got = df.predict(_dev(X), int8=True).cpu().numpy()
    df.check_status()
    pick = np.arange(0, rows, max(1, rows // 2000))
    _, sums = oracle.predict(forest, X[pick], class_sums=True)
    # a class without trees holds the initial value alone, as in the reference's generated
    # reduction (its header walker would leave it at 0)
    sums[:, 7] = forest.initial_value
    want = (sums.shape[1] - 1 - np.argmax(sums[:, ::-1], axis=1)).astype(np.float32)  # last maximum
    assert_predictions_close(got[pick], want, forest, sums)
    assert (want == 7).any() and (want != 7).any()     # the empty class wins on some rows only


def test_two_streams_share_one_forest():
    """Calls on one forest from two streams reuse the forest's tree-chunk scratch: the second
    stream must wait for the first call's second pass before its walk overwrites the sums."""
    from treebeard_b200 import kernels
    forest, X = small_config("c2", rows=8192)
    other = np.ascontiguousarray(X[::-1])
    want_a, want_b = oracle.predict(forest, X), oracle.predict(forest, other)
    df = kernels.DeviceForest(forest, representation="sparse", tree_chunks=4, batch_hint=len(X))
    a, b = _dev(X), _dev(other)
    s1, s2 = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    outs = []
    for it in range(6):
        with torch.cuda.stream(s1):
            oa = df.predict(a, stream=s1)
        with torch.cuda.stream(s2):
            ob = df.predict(b, stream=s2)
        outs.append((oa, ob))
    torch.cuda.synchronize()
    df.check_status()
    for oa, ob in outs:
        assert_predictions_close(oa.cpu().numpy(), want_a)
        assert_predictions_close(ob.cpu().numpy(), want_b)


def test_runner_rejects_buffers_on_different_sides(tmp_path):
    """Device buffers are an extension of the reference API: input and result must then both be
    on the device (a host result buffer would be written by the kernel)."""
    from treebeard_b200 import synth, treebeard
    from treebeard_b200.treebeard import treebeardAPI
    forest, X = small_config("c1")
    runner = treebeard.TreebeardInferenceRunner.FromForestArrays(forest, treebeard.CompilerOptions(1024, 1))
    host_out = np.zeros(1024, np.float32)
    dev_in, dev_out = _dev(X), torch.zeros(1024, device="cuda")
    with pytest.raises(treebeard.TreebeardRuntimeError, match="host memory"):
        treebeardAPI.RunInference(runner.inferenceRunner, dev_in.data_ptr(), host_out.ctypes.data)
    with pytest.raises(treebeard.TreebeardRuntimeError, match="device memory"):
        treebeardAPI.RunInference(runner.inferenceRunner, X.ctypes.data, dev_out.data_ptr())
    with pytest.raises(treebeard.TreebeardRuntimeError, match="shape"):
        runner.RunInference(X[:, :4].copy())
    assert_predictions_close(runner.RunInference(X), oracle.predict(forest, X))


def test_sixteen_bit_keys_refuse_what_they_do_not_cover():
    """Multiclass forests need rows narrow enough for the batch kernel."""
    from treebeard_b200 import kernels, synth
    wide = synth.generate_forest(40, 60, 6, 1800, 0.1, 0.1, synth.Marginal("normal", 1800), num_classes=3)
    with pytest.raises(kernels.TbkError):
        kernels.DeviceForest(wide, representation="auto", feature_bits=16)
    assert kernels.DeviceForest(wide, representation="auto").info().schedule.feature_bits == 32


def test_batched_key_kernel_multiclass_on_continuous_features():
    """Three classes over continuous features (ordinary keys, no lattice): an odd number of
    classes (the two walker sets get two and one), rare ties resolved exactly."""
    from treebeard_b200 import kernels, synth
    marg = synth.Marginal("normal", 10)
    forest = synth.generate_forest(77, 93, 6, 10, 0.1, 0.1, marg, num_classes=3)
    rng = np.random.Generator(np.random.PCG64(5))
    X = marg.sample_rows(rng, 40000)
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(500):
        g = split[(i * 37) % len(split)]
        X[(i * 31) % len(X), forest.feat[g]] = forest.thr[g]
    want, sums = oracle.predict(forest, X, class_sums=True)
    _, want_ids = oracle.predict(forest, X, leaf_ids=True)
    df = kernels.DeviceForest(forest, representation="auto", batch_hint=len(X))
    assert df.info().schedule.feature_bits == 16
    dX = _dev(X)
    assert_predictions_close(df.predict(dX).cpu().numpy(), want, forest, sums)
    assert np.array_equal(df.predict_leaf_ids(dX[:3000]).cpu().numpy(), want_ids[:3000])
    assert df.info().reserved[0] > 0          # key ties were hit and resolved exactly


@pytest.mark.parametrize("rows", [100003, 5000, 77])
def test_batched_key_kernel_multiclass(rows):
    """Multiclass forests on the batch kernel: classes laid out group by group, one walker set
    per class, arg-max on the fly with the reference's tie rule; int8 and fp32 class ids."""
    from treebeard_b200 import kernels
    forest, X = small_config("c4", rows=rows)
    X = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(2000):
        g = split[(i * 37) % len(split)]
        X[(i * 31) % len(X), forest.feat[g]] = forest.thr[g]
    for i in range(0, 2000, 3):                      # ... and values that are not whole numbers next to them
        g = split[(i * 37) % len(split)]
        X[(i * 31) % len(X), forest.feat[g]] += ((-1) ** i) * [1e-6, 1e-3, 0.5][i % 3]
    want, sums = oracle.predict(forest, X, class_sums=True)
    _, want_ids = oracle.predict(forest, X, leaf_ids=True)
    df = kernels.DeviceForest(forest, representation="auto", feature_bits=16, batch_hint=rows)
    info = df.info()
    assert info.schedule.feature_bits == 16 and info.threads_per_block == 704
    dX = _dev(X)
    got = df.predict(dX).cpu().numpy()
    df.check_status()
    assert_predictions_close(got, want, forest, sums)
    got8 = df.predict(dX, int8=True).cpu().numpy()
    assert got8.dtype == np.int8 and np.array_equal(got8, got.astype(np.int8))
    sub = slice(max(0, rows - 9001), rows)
    ids = df.predict_leaf_ids(dX[sub]).cpu().numpy()
    df.check_status()
    assert np.array_equal(ids, want_ids[sub])
    # per-class partial sums (what tree shards exchange) and the second pass over them
    part = df.predict_partial(dX)
    assert part.shape == (rows, forest.num_classes)
    assert np.allclose(part.cpu().numpy() + forest.initial_value, sums, rtol=1e-5, atol=1e-5) or \
        np.allclose(part.cpu().numpy(), sums, rtol=1e-5, atol=1e-5)
    assert_predictions_close(df.finalize(part).cpu().numpy(), want, forest, sums)


@pytest.mark.parametrize("name,layout", [("c2", dict(representation="sparse")),
                                         ("c2", dict(representation="auto", feature_bits=16)),
                                         ("c3", dict(representation="auto", feature_bits=16)),
                                         ("c5", dict(representation="auto", feature_bits=16))])
def test_expired_device_wait_is_reported_and_survivable(name, layout):
    """Failure drill on the host's initiative: the first tree stage of one launch is never
    copied, so the kernel's bounded wait gives up.  The launch must end by itself, the status
    check must report TBK_ERR_DEVICE_WAIT, and the next prediction must be correct again."""
    from treebeard_b200 import kernels
    forest, X = small_config(name)
    want = oracle.predict(forest, X)
    df = kernels.DeviceForest(forest, batch_hint=len(X), **layout)
    dX = _dev(X)
    assert_predictions_close(df.predict(dX).cpu().numpy(), want)
    df.check_status()
    df.expire_next_wait()
    df.predict(dX)                      # results undefined, but it returns
    torch.cuda.synchronize()
    with pytest.raises(kernels.TbkError) as err:
        df.check_status()
    assert err.value.status == 4        # TBK_ERR_DEVICE_WAIT
    assert_predictions_close(df.predict(dX).cpu().numpy(), want)
    df.check_status()
