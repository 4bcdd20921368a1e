"""TEST INFRASTRUCTURE -- Python face of the CPU oracle.

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the product package never does.

It (1) reads an XGBoost JSON model into flat numpy arrays following the
reference's front end (src/json/xgboostparser.h:94-114 base-score / objective
rules, :116-145 learner fields, :177-219 per-tree arrays; thresholds and leaf
values are narrowed double -> float as the reference's float ThresholdType does),
(2) calls the C restatement in walk.c (liboracle.so) and, when present, the shim
around the reference's unmodified header (_ref/libref_oracle.so).
"""
from __future__ import annotations

import ctypes
import json
import math
import os
import subprocess
from dataclasses import dataclass

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

IDENTITY, SIGMOID, SOFTMAX = 0, 1, 2


@dataclass
class FlatForest:
    """Forest as flat arrays; tree t owns nodes [tree_off[t], tree_off[t+1])."""
    tree_off: np.ndarray   # int64 [T+1]
    left: np.ndarray       # int32, -1 for a leaf
    right: np.ndarray      # int32, -1 for a leaf
    feat: np.ndarray       # int32
    thr: np.ndarray        # float32 (leaf value for leaves)
    class_id: np.ndarray   # int32 [T]
    num_classes: int
    transform: int
    initial_value: float
    num_features: int

    @property
    def num_trees(self) -> int:
        return len(self.tree_off) - 1


def forest_from_xgboost_dict(model: dict) -> FlatForest:
    learner = model["learner"]
    base_score = float(learner["learner_model_param"]["base_score"])
    objective = learner["objective"]["name"]
    if objective == "binary:logistic":
        initial, transform = -math.log(1.0 / base_score - 1.0), SIGMOID
    elif objective == "reg:squarederror":
        initial, transform = base_score, IDENTITY
    elif objective == "multi:softmax":
        initial, transform = base_score, SOFTMAX
    else:
        raise ValueError(f"unknown objective {objective}")
    num_classes = int(learner["learner_model_param"]["num_class"])
    booster = learner["gradient_booster"]["model"]
    trees = booster["trees"]
    assert int(booster["gbtree_model_param"]["num_trees"]) == len(trees)
    tree_info = booster["tree_info"]
    num_features = int(learner["learner_model_param"].get("num_feature", 0)) or len(
        learner.get("feature_types", []))
    offs, left, right, feat, thr = [0], [], [], [], []
    for tr in trees:
        n = int(tr["tree_param"]["num_nodes"])
        assert len(tr["left_children"]) == n
        left.append(np.asarray(tr["left_children"], dtype=np.int32))
        right.append(np.asarray(tr["right_children"], dtype=np.int32))
        feat.append(np.asarray(tr["split_indices"], dtype=np.int32))
        thr.append(np.asarray(tr["split_conditions"], dtype=np.float64).astype(np.float32))
        offs.append(offs[-1] + n)
    return FlatForest(np.asarray(offs, dtype=np.int64), np.concatenate(left),
                      np.concatenate(right), np.concatenate(feat), np.concatenate(thr),
                      np.asarray(tree_info, dtype=np.int32), num_classes, transform,
                      float(initial), num_features)


def load_xgboost_json(path: str) -> FlatForest:
    with open(path) as f:
        return forest_from_xgboost_dict(json.load(f))


# ----------------------------------------------------------------------------
# ctypes plumbing


class _CForest(ctypes.Structure):
    _fields_ = [("num_trees", ctypes.c_int64), ("tree_off", ctypes.c_void_p),
                ("left", ctypes.c_void_p), ("right", ctypes.c_void_p),
                ("feat", ctypes.c_void_p), ("thr", ctypes.c_void_p),
                ("class_id", ctypes.c_void_p), ("num_classes", ctypes.c_int32),
                ("transform", ctypes.c_int32), ("initial_value", ctypes.c_double),
                ("num_features", ctypes.c_int32)]


def reference_root() -> str | None:
    """Where the reference checkout lies: the TREEBEARD_REF environment variable, else the
    build container's mount point; None if neither exists."""
    for root in (os.environ.get("TREEBEARD_REF"), os.path.join(os.sep, "root", "reference")):
        if root and os.path.isdir(os.path.join(root, "src", "include")):
            return root
    return None


def build(ref_root: str | None = None) -> None:
    """Compile liboracle.so and, if a reference checkout is given (argument, else the
    TREEBEARD_REF environment variable) and exists, the shim around its header in _ref/."""
    ref_root = ref_root or reference_root()
    subprocess.run(["make", "-s", "-C", _HERE], check=True)
    if ref_root and os.path.isdir(os.path.join(ref_root, "src", "include")):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", f"REF={ref_root}"], check=True)


_lib = None
_ref = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build(None)
        _lib = ctypes.CDLL(path)
        _lib.tbo_sparse_build.restype = ctypes.c_void_p
        _lib.tbo_sparse_build.argtypes = [ctypes.c_void_p]
        _lib.tbo_sparse_free.argtypes = [ctypes.c_void_p]
    return _lib


def ref_lib():
    """The reference-header shim, or None if it was not built."""
    global _ref
    if _ref is None:
        path = os.path.join(_HERE, "_ref", "libref_oracle.so")
        if not os.path.exists(path):
            return None
        _ref = ctypes.CDLL(path)
        _ref.tbref_forest_create.restype = ctypes.c_void_p
    return _ref


def _ptr(a):
    return a.ctypes.data_as(ctypes.c_void_p)


def _cforest(f: FlatForest):
    keep = [np.ascontiguousarray(f.tree_off, np.int64), np.ascontiguousarray(f.left, np.int32),
            np.ascontiguousarray(f.right, np.int32), np.ascontiguousarray(f.feat, np.int32),
            np.ascontiguousarray(f.thr, np.float32), np.ascontiguousarray(f.class_id, np.int32)]
    c = _CForest(f.num_trees, *[a.ctypes.data for a in keep], f.num_classes, f.transform,
                 f.initial_value, f.num_features)
    return c, keep


def predict(f: FlatForest, rows: np.ndarray, leaf_ids: bool = False, class_sums: bool = False,
            tie_rule: int = 1):
    """Ground truth.  Returns preds [, leaf_ids int32 [n,T]] [, class_sums [n,C]]."""
    rows = np.ascontiguousarray(rows, dtype=np.float32)
    n = rows.shape[0]
    out = np.empty(n, np.float32)
    ids = np.empty((n, f.num_trees), np.int32) if leaf_ids else None
    cs = np.empty((n, max(f.num_classes, 1)), np.float32) if class_sums else None
    c, keep = _cforest(f)
    lib().tbo_predict(ctypes.byref(c), _ptr(rows), ctypes.c_int64(n),
                      ctypes.c_int64(rows.shape[1]), _ptr(out),
                      _ptr(ids) if leaf_ids else None, _ptr(cs) if class_sums else None,
                      ctypes.c_int32(tie_rule))
    res = [out]
    if leaf_ids:
        res.append(ids)
    if class_sums:
        res.append(cs)
    return res[0] if len(res) == 1 else tuple(res)


class CpuBaseline:
    """The reference's parallel CPU schedule restated (sparse layout, one row block
    per thread, tree loop outermost, fp32 sums)."""

    def __init__(self, f: FlatForest):
        c, keep = _cforest(f)
        self._h = lib().tbo_sparse_build(ctypes.byref(c))

    def predict(self, rows: np.ndarray, threads: int = 0) -> np.ndarray:
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        out = np.empty(rows.shape[0], np.float32)
        lib().tbo_cpu_baseline(ctypes.c_void_p(self._h), _ptr(rows),
                               ctypes.c_int64(rows.shape[0]), ctypes.c_int64(rows.shape[1]),
                               _ptr(out), ctypes.c_int32(threads))
        return out

    def __del__(self):
        if getattr(self, "_h", None):
            lib().tbo_sparse_free(ctypes.c_void_p(self._h))
            self._h = None


def max_threads() -> int:
    return int(lib().tbo_max_threads())


class RefForest:
    """The reference's own DecisionForest object, driven through the shim."""

    def __init__(self, f: FlatForest):
        r = ref_lib()
        if r is None:
            raise RuntimeError("oracle/_ref was not built")
        self.f = f
        keep = _cforest(f)[1]
        self._h = r.tbref_forest_create(
            ctypes.c_int64(f.num_trees), *[_ptr(a) for a in keep], ctypes.c_int32(f.num_classes),
            ctypes.c_int32(f.transform), ctypes.c_double(f.initial_value),
            ctypes.c_int32(f.num_features))

    def predict(self, rows: np.ndarray) -> np.ndarray:
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        out = np.empty(rows.shape[0], np.float32)
        ref_lib().tbref_predict(ctypes.c_void_p(self._h), _ptr(rows), ctypes.c_int64(rows.shape[0]),
                                ctypes.c_int64(rows.shape[1]), ctypes.c_int32(self.f.num_features),
                                _ptr(out))
        return out

    def tree_outputs(self, rows: np.ndarray) -> np.ndarray:
        rows = np.ascontiguousarray(rows, dtype=np.float32)
        out = np.empty((rows.shape[0], self.f.num_trees), np.float32)
        ref_lib().tbref_tree_outputs(ctypes.c_void_p(self._h), _ptr(rows),
                                     ctypes.c_int64(rows.shape[0]), ctypes.c_int64(rows.shape[1]),
                                     ctypes.c_int32(self.f.num_features), _ptr(out))
        return out

    def __del__(self):
        if getattr(self, "_h", None):
            ref_lib().tbref_forest_free(ctypes.c_void_p(self._h))
            self._h = None


def fp_equal(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """The reference's test tolerance (src/test/TestUtilsCommon.h:57-76):
    (a-b)^2 < max(1e-6, max(|a|,|b|)/1e8)."""
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    thr = np.maximum(1e-6, np.maximum(np.abs(a), np.abs(b)) / 1e8)
    return (a - b) ** 2 < thr
