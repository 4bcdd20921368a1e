"""Shared helpers for the parity tests."""
import numpy as np

from oracle import oracle
from treebeard_b200 import synth

# reduced sizes: the oracle finishes each in well under a second
SMALL = {"c1": dict(trees=None, rows=1024), "c2": dict(trees=200, rows=4096),
         "c3": dict(trees=48, rows=1500), "c4": dict(trees=260, rows=4096),
         "c5": dict(trees=48, rows=3000)}

REL_TOL, ABS_TOL = 1e-5, 1e-6   # prediction tolerance stated for this path


def small_config(name, rows=None, trees=None):
    s = SMALL[name]
    forest, marg, _ = synth.make_config(name, trees=trees if trees is not None else s["trees"])
    X = synth.config_rows(name, marg, rows if rows is not None else s["rows"])
    return forest, X


def assert_predictions_close(got, want, forest=None, class_sums=None):
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    if forest is not None and forest.num_classes > 0:
        # class ids must match except where the two best class sums are within rounding
        bad = got != want
        if bad.any():
            top2 = np.sort(class_sums[bad], axis=1)[:, -2:]
            margin = top2[:, 1] - top2[:, 0]
            assert (margin < 1e-5).all(), f"class id mismatch with margin {margin.max()}"
        return
    err = np.abs(got - want)
    ok = err <= ABS_TOL + REL_TOL * np.abs(want)
    assert ok.all(), f"max abs err {err.max()} at {err.argmax()}"


def golden_forest(npz):
    return oracle.FlatForest(npz["tree_off"], npz["left"], npz["right"], npz["feat"], npz["thr"],
                             npz["class_id"], int(npz["num_classes"]), int(npz["transform"]),
                             float(npz["initial_value"]), int(npz["num_features"]))
