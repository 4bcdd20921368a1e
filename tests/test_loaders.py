"""Native model front ends (XGBoost JSON, ONNX) checked on the host against the oracle's
own Python readers and the golden vectors."""
import os

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import small_config
from treebeard_b200 import synth, treebeard

# the reference's own ONNX model, where its checkout is mounted
REF_ONNX = os.path.join(oracle.reference_root() or "", "onnx_models", "abalone_onnx_model_save.onnx")


def same_function(a, b, X):
    """Two forests describe the same function on X: identical predictions (node numbering
    may differ between loaders)."""
    return np.array_equal(oracle.predict(a, X), oracle.predict(b, X))


@pytest.mark.parametrize("stem", ["TestModel_Size2_1", "TestModel_Size4_10", "leftheavy_xgb_model",
                                  "rightandleftheavy_xgb_model"])
def test_native_xgboost_loader_matches_python_reader(stem, golden_dir):
    path = os.path.join(golden_dir, stem + ".json")
    native = treebeard.LoadForest(path, "xgboost_json")
    ref = oracle.load_xgboost_json(path)
    for name in ("tree_off", "left", "right", "thr"):
        assert np.array_equal(getattr(native, name), getattr(ref, name)), name
    split = ref.left >= 0
    assert np.array_equal(native.feat[split], ref.feat[split])
    assert native.num_features == ref.num_features and native.transform == ref.transform
    assert native.initial_value == pytest.approx(ref.initial_value)
    z = np.load(os.path.join(golden_dir, stem + ".npz"))
    assert oracle.fp_equal(oracle.predict(native, z["rows"]), z["expected"]).all()


def test_native_xgboost_loader_objectives(tmp_path):
    for name in ("c2", "c4"):
        forest, X = small_config(name, rows=64, trees=52)
        path = str(tmp_path / f"{name}.json")
        synth.save_xgboost_json(forest, path)
        native = treebeard.LoadForest(path, "xgboost_json")
        assert native.num_classes == forest.num_classes and native.transform == forest.transform
        assert native.initial_value == pytest.approx(forest.initial_value)
        assert np.array_equal(native.class_id, forest.class_id)
        assert same_function(native, forest, X)


@pytest.mark.parametrize("mode", ["BRANCH_LT", "BRANCH_LEQ", "BRANCH_GEQ", "BRANCH_GT"])
@pytest.mark.parametrize("packed", [False, True])
def test_onnx_loader_every_comparison_mode(mode, packed, tmp_path):
    forest, X = small_config("c2", rows=300, trees=40)
    # rows that sit exactly on thresholds: the <= / > rewrites must not move them
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(200):
        g = split[(i * 13) % len(split)]
        X[i, forest.feat[g]] = forest.thr[g]
    path = str(tmp_path / "m.onnx")
    synth.save_onnx(forest, path, mode=mode, packed=packed)
    native = treebeard.LoadForest(path, "onnx_file", forest.num_features)
    assert native.num_trees == forest.num_trees and native.num_nodes == forest.num_nodes
    assert native.transform == synth.SIGMOID and native.num_classes == 0
    want, want_ids = oracle.predict(forest, X, leaf_ids=True)
    got = oracle.predict(native, X)
    assert np.array_equal(got, want)


def test_onnx_classifier(tmp_path):
    forest, X = small_config("c4", rows=200, trees=52)
    path = str(tmp_path / "c.onnx")
    synth.save_onnx(forest, path)
    native = treebeard.LoadForest(path, "onnx_file", 16)
    assert native.num_classes == 26 and native.transform == synth.SOFTMAX
    assert np.array_equal(native.class_id, forest.class_id)
    assert same_function(native, forest, X)


def test_onnx_errors(tmp_path):
    bad = tmp_path / "bad.onnx"
    bad.write_bytes(b"\x08\x07\x12\x03abc")
    with pytest.raises(treebeard.TreebeardRuntimeError, match="graph"):
        treebeard.LoadForest(str(bad), "onnx_file")
    with pytest.raises(treebeard.TreebeardRuntimeError, match="cannot open"):
        treebeard.LoadForest(str(tmp_path / "none.onnx"), "onnx_file")


@pytest.mark.skipif(not os.path.exists(REF_ONNX), reason="reference checkout not mounted")
def test_reference_abalone_onnx_against_its_csv():
    native = treebeard.LoadForest(REF_ONNX, "onnx_file", 8)
    data = np.loadtxt(REF_ONNX + ".csv", delimiter=",")
    rows, expected = data[:, :-1].astype(np.float32), data[:, -1].astype(np.float32)
    assert native.num_features == 8 and native.num_classes == 0
    got = oracle.predict(native, rows)
    assert oracle.fp_equal(got, expected).all()


def test_abalone_golden_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "abalone_onnx.npz"))
    from tests.helpers import golden_forest
    forest = golden_forest(z)
    assert oracle.fp_equal(oracle.predict(forest, z["rows"]), z["expected"]).all()
