"""Seeded synthetic forests and inputs for the five benchmark configurations.

The configurations name no public dataset; forests and feature matrices are drawn
from ``numpy.random.Generator(PCG64(seed))`` with the shapes and value
distributions each configuration states.  Forests can be written in the XGBoost
JSON (version [1, 4, 0]) schema that the reference's loader reads
(src/json/xgboostparser.h:116-219) and its own random-model writer emits
(src/utils/RandomTreeGenerator.cpp:83-167): per tree ``left_children``,
``right_children``, ``parents`` (root: 2147483647), ``split_indices``,
``split_conditions`` (leaf value for leaves), ``base_weights``, ``default_left``,
``tree_param.{num_feature,num_nodes}``; ``tree_info`` = class id per tree.

Tree generator (seed, T trees, D decision levels, F features, leaf probability p):
a node at level d is a leaf if d == D, else if d > 0 and U[0,1) < p; otherwise it
splits on a feature ~ UniformInt[0, F) at an fp32 threshold drawn from that
feature's input marginal.  Nodes are numbered in level order, children adjacent.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field

import numpy as np

IDENTITY, SIGMOID, SOFTMAX = 0, 1, 2
_OBJECTIVE = {IDENTITY: "reg:squarederror", SIGMOID: "binary:logistic", SOFTMAX: "multi:softmax"}


@dataclass
class ForestArrays:
    """Forest as flat arrays; tree t owns nodes [tree_off[t], tree_off[t+1]).
    ``left``/``right`` are node indices inside the tree, -1 for a leaf; ``thr`` is
    the split threshold or, for a leaf, the leaf value."""
    tree_off: np.ndarray
    left: np.ndarray
    right: np.ndarray
    feat: np.ndarray
    thr: np.ndarray
    class_id: np.ndarray
    num_classes: int
    transform: int
    initial_value: float
    num_features: int
    base_score: float = 0.5

    @property
    def num_trees(self) -> int:
        return len(self.tree_off) - 1

    @property
    def num_nodes(self) -> int:
        return int(self.tree_off[-1])

    def tree_slice(self, t0: int, t1: int) -> "ForestArrays":
        """Trees [t0, t1) as a forest of their own (tree sharding)."""
        a, b = int(self.tree_off[t0]), int(self.tree_off[t1])
        return ForestArrays(self.tree_off[t0:t1 + 1] - a, self.left[a:b], self.right[a:b],
                            self.feat[a:b], self.thr[a:b], self.class_id[t0:t1], self.num_classes,
                            self.transform, self.initial_value, self.num_features, self.base_score)


# ---------------------------------------------------------------------------
# input marginals


@dataclass
class Marginal:
    """Per-feature input distribution; ``kind``: 'uniform01', 'normal', 'int16',
    'mix' (each feature is N(0,1) or U[-5,5], decided by a seeded coin)."""
    kind: str
    num_features: int
    seed: int = 0
    uniform_cols: np.ndarray = field(default=None, repr=False)

    def __post_init__(self):
        if self.kind == "mix":
            coin = np.random.Generator(np.random.PCG64(self.seed + 7919))
            self.uniform_cols = coin.random(self.num_features) < 0.5

    def sample_for_features(self, rng, feat: np.ndarray) -> np.ndarray:
        n = len(feat)
        if self.kind == "uniform01":
            return rng.random(n, dtype=np.float32)
        if self.kind == "normal":
            return rng.standard_normal(n, dtype=np.float32)
        if self.kind == "int16":
            return rng.integers(0, 16, n).astype(np.float32)
        if self.kind == "mix":
            nrm = rng.standard_normal(n, dtype=np.float32)
            uni = (rng.random(n, dtype=np.float32) * np.float32(10.0) - np.float32(5.0))
            return np.where(self.uniform_cols[feat], uni, nrm).astype(np.float32)
        raise ValueError(self.kind)

    def sample_rows(self, rng, n_rows: int) -> np.ndarray:
        F = self.num_features
        if self.kind == "uniform01":
            return rng.random((n_rows, F), dtype=np.float32)
        if self.kind == "normal":
            return rng.standard_normal((n_rows, F), dtype=np.float32)
        if self.kind == "int16":
            return rng.integers(0, 16, (n_rows, F), dtype=np.int8).astype(np.float32)
        if self.kind == "mix":
            x = rng.standard_normal((n_rows, F), dtype=np.float32)
            cols = np.nonzero(self.uniform_cols)[0]
            x[:, cols] = rng.random((n_rows, len(cols)), dtype=np.float32) * np.float32(10.0) \
                - np.float32(5.0)
            return x
        raise ValueError(self.kind)


# ---------------------------------------------------------------------------
# forest generator


def generate_forest(seed: int, T: int, D: int, F: int, p: float, leaf_sigma: float,
                    marginal: Marginal, transform: int = IDENTITY, num_classes: int = 0,
                    base_score: float = 0.5) -> ForestArrays:
    rng = np.random.Generator(np.random.PCG64(seed))
    level_tree = np.arange(T, dtype=np.int64)
    lv_tree, lv_leaf, lv_feat, lv_thr = [], [], [], []
    for d in range(D + 1):
        n = len(level_tree)
        if d == D:
            is_leaf = np.ones(n, bool)
        elif d == 0 or p <= 0.0:
            is_leaf = np.zeros(n, bool)
        else:
            is_leaf = rng.random(n) < p
        ns = int(n - is_leaf.sum())
        feat = np.zeros(n, np.int32)
        thr = np.empty(n, np.float32)
        sf = rng.integers(0, F, ns).astype(np.int32)
        feat[~is_leaf] = sf
        thr[~is_leaf] = marginal.sample_for_features(rng, sf)
        thr[is_leaf] = (rng.standard_normal(n - ns) * leaf_sigma).astype(np.float32)
        lv_tree.append(level_tree); lv_leaf.append(is_leaf); lv_feat.append(feat); lv_thr.append(thr)
        level_tree = np.repeat(level_tree[~is_leaf], 2)
        if len(level_tree) == 0:
            break
    L = len(lv_tree)
    cnt = np.stack([np.bincount(t, minlength=T) for t in lv_tree])          # [L, T]
    lvl_start = np.cumsum(cnt, axis=0) - cnt                                 # start of level in tree
    tree_off = np.zeros(T + 1, np.int64)
    tree_off[1:] = np.cumsum(cnt.sum(axis=0))
    total = int(tree_off[-1])
    left = np.full(total, -1, np.int32); right = np.full(total, -1, np.int32)
    feat = np.zeros(total, np.int32); thr = np.empty(total, np.float32)
    for d in range(L):
        t = lv_tree[d]
        first = np.cumsum(cnt[d]) - cnt[d]                                   # first position of tree
        local = lvl_start[d][t] + (np.arange(len(t)) - first[t])
        g = tree_off[t] + local
        feat[g] = lv_feat[d]; thr[g] = lv_thr[d]
        split = ~lv_leaf[d]
        if split.any():
            k = np.arange(int(split.sum()))
            ts = t[split]
            first_n = np.cumsum(cnt[d + 1]) - cnt[d + 1]
            lchild = lvl_start[d + 1][ts] + (2 * k - first_n[ts])
            left[g[split]] = lchild.astype(np.int32)
            right[g[split]] = (lchild + 1).astype(np.int32)
    class_id = (np.arange(T) % num_classes).astype(np.int32) if num_classes > 0 \
        else np.zeros(T, np.int32)
    if transform == SIGMOID:
        initial = -np.log(1.0 / base_score - 1.0)
    else:
        initial = base_score
    return ForestArrays(tree_off, left, right, feat, thr, class_id, num_classes, transform,
                        float(initial), F, base_score)


def generate_rows(seed: int, marginal: Marginal, n_rows: int) -> np.ndarray:
    rng = np.random.Generator(np.random.PCG64(seed))
    return marginal.sample_rows(rng, n_rows)


# ---------------------------------------------------------------------------
# the five configurations

CONFIGS = {
    # name: trees, levels, features, leaf prob, leaf sigma, marginal, transform, classes, rows
    "c1": dict(T=100, D=6, F=8, p=0.0, sigma=0.1, kind="uniform01", transform=IDENTITY,
               classes=0, rows=1024, forest_seed=1001, row_seed=2001,
               desc="regression T=100 D=6 complete F=8"),
    "c2": dict(T=1000, D=8, F=28, p=0.15, sigma=0.05, kind="normal", transform=SIGMOID,
               classes=0, rows=1048576, forest_seed=1002, row_seed=2002,
               desc="binary classifier T=1000 D=8 p=0.15 F=28"),
    "c3": dict(T=1000, D=8, F=2000, p=0.0, sigma=0.02, kind="normal", transform=IDENTITY,
               classes=0, rows=262144, forest_seed=1003, row_seed=2003,
               desc="wide dense regressor T=1000 D=8 complete F=2000"),
    "c4": dict(T=2600, D=8, F=16, p=0.1, sigma=0.1, kind="int16", transform=SOFTMAX,
               classes=26, rows=1048576, forest_seed=1004, row_seed=2004,
               desc="multiclass 26x100 D=8 p=0.1 F=16"),
    "c5": dict(T=16000, D=12, F=128, p=0.05, sigma=0.01, kind="mix", transform=IDENTITY,
               classes=0, rows=4194304, forest_seed=1005, row_seed=2005,
               desc="large forest T=16000 D=12 p=0.05 F=128"),
}


def make_config(name: str, trees: int | None = None, rows: int | None = None,
                row_seed_offset: int = 0):
    """(forest, marginal, n_rows) for a configuration; ``trees`` / ``rows`` override
    the full sizes (parity tests use reduced ones).  For the multiclass configuration
    ``trees`` is rounded to a multiple of the class count."""
    c = CONFIGS[name]
    T = c["T"] if trees is None else trees
    if c["classes"] > 0:
        T = max(c["classes"], (T // c["classes"]) * c["classes"])
    marg = Marginal(c["kind"], c["F"], seed=c["forest_seed"])
    forest = generate_forest(c["forest_seed"], T, c["D"], c["F"], c["p"], c["sigma"], marg,
                             c["transform"], c["classes"])
    return forest, marg, (c["rows"] if rows is None else rows)


def config_rows(name: str, marginal: Marginal, n_rows: int, offset: int = 0) -> np.ndarray:
    return generate_rows(CONFIGS[name]["row_seed"] + offset, marginal, n_rows)


# ---------------------------------------------------------------------------
# XGBoost JSON writer


def to_xgboost_dict(f: ForestArrays) -> dict:
    trees = []
    for t in range(f.num_trees):
        a, b = int(f.tree_off[t]), int(f.tree_off[t + 1])
        n = b - a
        l, r = f.left[a:b], f.right[a:b]
        parents = np.full(n, 2147483647, np.int64)
        idx = np.arange(n)
        parents[l[l >= 0]] = idx[l >= 0]
        parents[r[r >= 0]] = idx[r >= 0]
        zeros = [0.0] * n
        trees.append({
            "id": t,
            "tree_param": {"num_deleted": "0", "num_feature": str(f.num_features),
                           "num_nodes": str(n), "size_leaf_vector": "0"},
            "loss_changes": zeros, "sum_hessian": zeros, "base_weights": zeros,
            "default_left": [False] * n, "categories": [], "categories_nodes": [],
            "categories_segments": [], "categories_sizes": [],
            "left_children": l.tolist(), "right_children": r.tolist(),
            "parents": parents.tolist(), "split_indices": f.feat[a:b].tolist(),
            "split_conditions": [float(v) for v in f.thr[a:b]],
        })
    return {
        "version": [1, 4, 0],
        "learner": {
            "attributes": {},
            "feature_types": ["float"] * f.num_features,
            "learner_model_param": {"base_score": repr(float(f.base_score)),
                                    "num_class": str(f.num_classes),
                                    "num_feature": str(f.num_features)},
            "objective": {"name": _OBJECTIVE[f.transform]},
            "gradient_booster": {
                "name": "gbtree",
                "model": {"gbtree_model_param": {"num_trees": str(f.num_trees),
                                                 "size_leaf_vector": "0"},
                          "tree_info": f.class_id.tolist(), "trees": trees},
            },
        },
    }


def save_xgboost_json(f: ForestArrays, path: str) -> None:
    with open(path, "w") as fh:
        json.dump(to_xgboost_dict(f), fh)
