"""Regenerates the golden fixtures in this folder from the reference checkout.

Run in a container that has the reference mounted (--ref, default: $TREEBEARD_REF):

    python tests/golden/make_golden.py [--ref <reference checkout>]

For every model whose JSON *and* golden CSV exist in the reference's
``xgb_models`` tree (CSV rows = features..., XGBoost's prediction; consumed by the
reference's ValidateModuleOutputAgainstCSVdata, src/test/TestUtilsCommon.h:166-222)
it (1) checks the CPU oracle -- and the shim around the reference's own header,
when built -- against ALL rows of the CSV under the reference's FPEqual tolerance
and records the outcome in ``manifest.json``, (2) stores a compact fixture that
travels with the repository:

  * benchmark models (higgs, airline, year_prediction_msd): ``<name>.npz`` with
    the flat forest arrays, the first ROWS rows and their expected predictions;
  * a few Random_{1,2,4}Tree models and the three hand-shaped models:
    ``<name>.json`` (the model, trimmed to the fields a loader reads) plus
    ``<name>.npz`` with rows / expected predictions (hand-shaped models have no
    CSV; their expectations come from the reference header via oracle/_ref).
"""
import argparse
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "..", ".."))
from oracle import oracle  # noqa: E402

ROWS = 256


def read_csv(path):
    data = np.loadtxt(path, delimiter=",", dtype=np.float64)
    return data[:, :-1].astype(np.float32), data[:, -1].astype(np.float32)


def trim(model):
    for tr in model["learner"]["gradient_booster"]["model"]["trees"]:
        for k in ("loss_changes", "sum_hessian", "categories", "categories_nodes",
                  "categories_segments", "categories_sizes", "split_type"):
            tr.pop(k, None)
    return model


def check(forest, rows, expected):
    got = oracle.predict(forest, rows)
    res = {"rows": int(len(rows)), "oracle_pass": int(oracle.fp_equal(got, expected).sum()),
           "oracle_max_abs_diff": float(np.abs(got - expected).max())}
    if oracle.ref_lib() is not None:
        ref = oracle.RefForest(forest).predict(rows)
        res["ref_header_pass"] = int(oracle.fp_equal(ref, expected).sum())
        res["oracle_vs_ref_header_max_abs_diff"] = float(np.abs(got - ref).max())
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=oracle.reference_root(), required=oracle.reference_root() is None)
    args = ap.parse_args()
    xgb = os.path.join(args.ref, "xgb_models")
    manifest = {}

    for name in ("higgs", "airline", "year_prediction_msd"):
        mpath = os.path.join(xgb, f"{name}_xgb_model_save.json")
        forest = oracle.load_xgboost_json(mpath)
        entry = {}
        rows0 = exp0 = None
        for suffix in (".csv", ".test.sampled.csv"):
            cpath = mpath + suffix
            if not os.path.exists(cpath):
                continue
            rows, exp = read_csv(cpath)
            entry[os.path.basename(cpath)] = check(forest, rows, exp)
            if rows0 is None:
                rows0, exp0 = rows, exp
        np.savez_compressed(os.path.join(HERE, f"{name}.npz"), tree_off=forest.tree_off,
                            left=forest.left, right=forest.right, feat=forest.feat, thr=forest.thr,
                            class_id=forest.class_id, num_classes=forest.num_classes,
                            transform=forest.transform, initial_value=forest.initial_value,
                            num_features=forest.num_features, rows=rows0[:ROWS],
                            expected=exp0[:ROWS])
        manifest[name] = entry

    for folder, picks in (("Random_1Tree", ("TestModel_Size1_1", "TestModel_Size1_8")),
                          ("Random_2Tree", ("TestModel_Size2_1", "TestModel_Size2_13")),
                          ("Random_4Tree", ("TestModel_Size4_1", "TestModel_Size4_10"))):
        # every model of the folder is checked; only the picks are stored
        for fn in sorted(os.listdir(os.path.join(xgb, "test", folder))):
            if not fn.endswith(".json"):
                continue
            mpath = os.path.join(xgb, "test", folder, fn)
            if not os.path.exists(mpath + ".csv"):
                continue
            forest = oracle.load_xgboost_json(mpath)
            rows, exp = read_csv(mpath + ".csv")
            manifest[f"{folder}/{fn}"] = check(forest, rows, exp)
            stem = fn[:-5]
            if stem in picks:
                with open(mpath) as fh:
                    model = trim(json.load(fh))
                with open(os.path.join(HERE, f"{stem}.json"), "w") as fh:
                    json.dump(model, fh, separators=(",", ":"))
                np.savez_compressed(os.path.join(HERE, f"{stem}.npz"), rows=rows[:ROWS],
                                    expected=exp[:ROWS])

    rng = np.random.Generator(np.random.PCG64(99))
    for stem in ("leftheavy_xgb_model", "rightheavy_xgb_model", "rightandleftheavy_xgb_model"):
        mpath = os.path.join(xgb, "test", stem + ".json")
        forest = oracle.load_xgboost_json(mpath)
        rows = (rng.random((ROWS, max(forest.num_features, 1)), dtype=np.float32) * 2 - 1) * 2
        exp = oracle.RefForest(forest).predict(rows) if oracle.ref_lib() is not None \
            else oracle.predict(forest, rows)
        with open(mpath) as fh:
            model = trim(json.load(fh))
        with open(os.path.join(HERE, f"{stem}.json"), "w") as fh:
            json.dump(model, fh, separators=(",", ":"))
        np.savez_compressed(os.path.join(HERE, f"{stem}.npz"), rows=rows, expected=exp)
        manifest[stem] = {"rows": ROWS, "expected_from": "reference header via oracle/_ref"}

    # ONNX: the reference's abalone regressor (consumed by its src/test/ONNXTests.cpp:32).
    # The file is parsed with this repository's native ONNX front end; the CSV pins the
    # result, and the forest is stored as flat arrays.
    onnx_path = os.path.join(args.ref, "onnx_models", "abalone_onnx_model_save.onnx")
    if os.path.exists(onnx_path):
        from treebeard_b200 import treebeard
        forest = treebeard.LoadForest(onnx_path, "onnx_file", 8)
        rows, exp = read_csv(onnx_path + ".csv")
        manifest["abalone_onnx"] = check(forest, rows, exp)
        np.savez_compressed(os.path.join(HERE, "abalone_onnx.npz"), tree_off=forest.tree_off,
                            left=forest.left, right=forest.right, feat=forest.feat, thr=forest.thr,
                            class_id=forest.class_id, num_classes=forest.num_classes,
                            transform=forest.transform, initial_value=forest.initial_value,
                            num_features=forest.num_features, rows=rows[:ROWS], expected=exp[:ROWS])

    with open(os.path.join(HERE, "manifest.json"), "w") as fh:
        json.dump(manifest, fh, indent=1, sort_keys=True)
    bad = {k: v for k, v in manifest.items()
           for vv in ([v] if "rows" in v else v.values())
           if "oracle_pass" in vv and vv["oracle_pass"] != vv["rows"]}
    print("models checked:", len(manifest), "with failures:", len(bad))
    for k, v in bad.items():
        print("  FAIL", k, v)


if __name__ == "__main__":
    main()
