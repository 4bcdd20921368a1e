"""The CPU oracle against the reference's golden vectors and against the reference's own
header (when oracle/_ref was built)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import SMALL, golden_forest, small_config
from treebeard_b200 import synth


@pytest.mark.parametrize("model", ["higgs", "airline", "year_prediction_msd"])
def test_benchmark_models_match_golden_csv(model, golden_dir):
    z = np.load(os.path.join(golden_dir, model + ".npz"))
    got = oracle.predict(golden_forest(z), z["rows"])
    assert oracle.fp_equal(got, z["expected"]).all()


@pytest.mark.parametrize("stem", ["TestModel_Size1_1", "TestModel_Size1_8", "TestModel_Size2_1",
                                  "TestModel_Size2_13", "TestModel_Size4_1", "TestModel_Size4_10",
                                  "leftheavy_xgb_model", "rightheavy_xgb_model",
                                  "rightandleftheavy_xgb_model"])
def test_json_models_match_golden(stem, golden_dir):
    forest = oracle.load_xgboost_json(os.path.join(golden_dir, stem + ".json"))
    z = np.load(os.path.join(golden_dir, stem + ".npz"))
    got = oracle.predict(forest, z["rows"])
    assert oracle.fp_equal(got, z["expected"]).all()


def test_manifest_records_full_csv_agreement(golden_dir):
    with open(os.path.join(golden_dir, "manifest.json")) as fh:
        manifest = json.load(fh)
    checked = 0
    for entry in manifest.values():
        for rec in ([entry] if "rows" in entry else entry.values()):
            if "oracle_pass" in rec:
                assert rec["oracle_pass"] == rec["rows"]
                assert rec.get("ref_header_pass", rec["rows"]) == rec["rows"]
                checked += 1
    assert checked >= 80


@pytest.mark.parametrize("name", list(SMALL))
def test_restatement_equals_reference_header(name):
    if oracle.ref_lib() is None:
        pytest.skip("oracle/_ref not built (needs the reference checkout)")
    forest, X = small_config(name, rows=400)
    got = oracle.predict(forest, X, tie_rule=0)
    ref = oracle.RefForest(forest).predict(X)
    assert np.array_equal(got, ref)


@pytest.mark.parametrize("name", list(SMALL))
def test_cpu_baseline_agrees_with_ground_truth(name):
    forest, X = small_config(name, rows=500)
    want, sums = oracle.predict(forest, X, class_sums=True)
    got = oracle.CpuBaseline(forest).predict(X, 2)
    if forest.num_classes:
        bad = got != want
        top2 = np.sort(sums[bad], axis=1)[:, -2:]
        assert ((top2[:, 1] - top2[:, 0]) < 1e-5).all()
    else:
        assert np.allclose(got, want, rtol=1e-5, atol=1e-6)


def test_leaf_ids_are_leaves_and_consistent():
    forest, X = small_config("c2", rows=200)
    preds, ids = oracle.predict(forest, X, leaf_ids=True)
    g = forest.tree_off[:-1][None, :] + ids
    assert (forest.left[g] == -1).all() and (forest.right[g] == -1).all()
    raw = forest.initial_value + forest.thr[g].astype(np.float64).sum(axis=1)
    assert np.allclose(1.0 / (1.0 + np.exp(-raw)), preds, rtol=1e-6, atol=1e-7)


def test_generator_shapes_and_determinism():
    f1, _, _ = synth.make_config("c1")
    f2, _, _ = synth.make_config("c1")
    assert f1.num_trees == 100 and f1.num_nodes == 100 * 127 and f1.num_features == 8
    assert np.array_equal(f1.thr, f2.thr) and np.array_equal(f1.feat, f2.feat)
    f4, _, _ = synth.make_config("c4", trees=260)
    assert f4.num_classes == 26 and (f4.class_id == np.arange(260) % 26).all()
    f3, m3, _ = synth.make_config("c3", trees=4)
    assert f3.num_nodes == 4 * 511
    # every tree is a proper binary tree in level order with adjacent children
    for f in (f1, f4, f3):
        split = f.left >= 0
        assert (f.right[split] == f.left[split] + 1).all()
        assert ((f.left < 0) == (f.right < 0)).all()


def test_xgboost_json_round_trip(tmp_path):
    forest, X = small_config("c4", rows=100, trees=52)
    path = str(tmp_path / "m.json")
    synth.save_xgboost_json(forest, path)
    back = oracle.load_xgboost_json(path)
    assert np.array_equal(back.thr, forest.thr) and np.array_equal(back.left, forest.left)
    assert back.num_classes == 26 and back.transform == synth.SOFTMAX
    assert np.array_equal(oracle.predict(back, X), oracle.predict(forest, X))
