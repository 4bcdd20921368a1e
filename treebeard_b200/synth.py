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


def node_depths(f: ForestArrays) -> np.ndarray:
    """Decision levels above every node (root 0), for forests whose nodes are numbered in
    level order with parents before children (what generate_forest produces)."""
    depth = np.zeros(f.num_nodes, np.int32)
    base = np.repeat(f.tree_off[:-1], np.diff(f.tree_off))
    split = np.nonzero(f.left >= 0)[0]
    # parents precede their children inside a tree, so one pass per level settles everything
    frontier = split[depth[split] == 0]
    frontier = frontier[np.isin(frontier, f.tree_off[:-1])]
    while len(frontier):
        kids = np.concatenate([base[frontier] + f.left[frontier], base[frontier] + f.right[frontier]])
        depth[kids] = np.concatenate([depth[frontier], depth[frontier]]) + 1
        frontier = kids[f.left[kids] >= 0]
    return depth


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


# ---------------------------------------------------------------------------
# ONNX writer (TreeEnsembleRegressor / TreeEnsembleClassifier, protobuf wire format)


def _varint(v: int) -> bytes:
    v &= (1 << 64) - 1
    out = bytearray()
    while True:
        b = v & 0x7F
        v >>= 7
        if v:
            out.append(b | 0x80)
        else:
            out.append(b)
            return bytes(out)


def _field(num: int, wire: int, payload: bytes) -> bytes:
    return _varint((num << 3) | wire) + payload


def _bytes_field(num: int, data: bytes) -> bytes:
    return _field(num, 2, _varint(len(data)) + data)


def _attr(name: str, *, f=None, i=None, s=None, floats=None, ints=None, strings=None,
          packed: bool = False) -> bytes:
    import struct
    body = _bytes_field(1, name.encode())
    if f is not None:
        body += _field(2, 5, struct.pack("<f", f)) + _field(20, 0, _varint(1))
    if i is not None:
        body += _field(3, 0, _varint(i)) + _field(20, 0, _varint(2))
    if s is not None:
        body += _bytes_field(4, s.encode()) + _field(20, 0, _varint(3))
    if floats is not None:
        arr = np.asarray(floats, np.float32)
        if packed:
            body += _bytes_field(7, arr.tobytes())
        else:
            body += b"".join(_field(7, 5, struct.pack("<f", x)) for x in arr)
        body += _field(20, 0, _varint(6))
    if ints is not None:
        if packed:
            body += _bytes_field(8, b"".join(_varint(int(x)) for x in ints))
        else:
            body += b"".join(_field(8, 0, _varint(int(x))) for x in ints)
        body += _field(20, 0, _varint(7))
    if strings is not None:
        body += b"".join(_bytes_field(9, x.encode()) for x in strings) + _field(20, 0, _varint(8))
    return _bytes_field(5, body)


def to_onnx_bytes(f: ForestArrays, mode: str = "BRANCH_LT", packed: bool = False) -> bytes:
    """Serialises the forest as a single-node ONNX graph.  ``mode`` picks the comparison the
    file states; thresholds and branches are rewritten so that every mode describes the SAME
    function as the forest's "x < t goes left" (x <= t' with t' the float below t, and the
    negated modes with the branches exchanged)."""
    classifier = f.num_classes > 0
    tree_ids, node_ids, feats, values, modes, true_ids, false_ids = [], [], [], [], [], [], []
    w_tree, w_node, w_ids, w_val = [], [], [], []
    swap = mode in ("BRANCH_GEQ", "BRANCH_GT")
    lower = mode in ("BRANCH_LEQ", "BRANCH_GT")
    for t in range(f.num_trees):
        a, b = int(f.tree_off[t]), int(f.tree_off[t + 1])
        for n in range(b - a):
            leaf = f.left[a + n] < 0
            thr = np.float32(f.thr[a + n])
            if not leaf and lower:
                thr = np.nextafter(thr, np.float32(-np.inf))
            lchild, rchild = int(f.left[a + n]), int(f.right[a + n])
            tree_ids.append(t); node_ids.append(n)
            feats.append(0 if leaf else int(f.feat[a + n]))
            values.append(0.0 if leaf else float(thr))
            modes.append("LEAF" if leaf else mode)
            true_ids.append(0 if leaf else (rchild if swap else lchild))
            false_ids.append(0 if leaf else (lchild if swap else rchild))
            if leaf:
                w_tree.append(t); w_node.append(n)
                w_ids.append(int(f.class_id[t]) if classifier else 0)
                w_val.append(float(f.thr[a + n]))
    post = {IDENTITY: "NONE", SIGMOID: "LOGISTIC", SOFTMAX: "SOFTMAX"}[f.transform]
    kw = dict(packed=packed)
    attrs = [
        _attr("nodes_treeids", ints=tree_ids, **kw), _attr("nodes_nodeids", ints=node_ids, **kw),
        _attr("nodes_featureids", ints=feats, **kw), _attr("nodes_values", floats=values, **kw),
        _attr("nodes_modes", strings=modes), _attr("nodes_truenodeids", ints=true_ids, **kw),
        _attr("nodes_falsenodeids", ints=false_ids, **kw),
        _attr("nodes_missing_value_tracks_true", ints=[0] * len(node_ids), **kw),
        _attr("post_transform", s=post),
    ]
    pre = "class_" if classifier else "target_"
    attrs += [_attr(pre + "treeids", ints=w_tree, **kw), _attr(pre + "nodeids", ints=w_node, **kw),
              _attr(pre + "ids", ints=w_ids, **kw), _attr(pre + "weights", floats=w_val, **kw)]
    if classifier:
        attrs += [_attr("classlabels_int64s", ints=list(range(f.num_classes)), **kw),
                  _attr("base_values", floats=[f.initial_value] * f.num_classes, **kw)]
        op = "TreeEnsembleClassifier"
    else:
        attrs += [_attr("n_targets", i=1), _attr("base_values", floats=[f.initial_value], **kw)]
        op = "TreeEnsembleRegressor"
    node = (_bytes_field(1, b"X") + _bytes_field(2, b"Y") + _bytes_field(3, b"ensemble") +
            _bytes_field(4, op.encode()) + b"".join(attrs) + _bytes_field(7, b"ai.onnx.ml"))
    graph = _bytes_field(1, node) + _bytes_field(2, b"forest")
    return _field(1, 0, _varint(7)) + _bytes_field(2, b"treebeard_b200") + _bytes_field(7, graph)


def save_onnx(f: ForestArrays, path: str, mode: str = "BRANCH_LT", packed: bool = False) -> None:
    with open(path, "wb") as fh:
        fh.write(to_onnx_bytes(f, mode, packed))
