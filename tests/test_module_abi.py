"""The module-side symbols that the reference's runner resolves by name (include/tbk_module.h):
Init_Model / Init_Offsets / Init_Lengths / Init_ClassIds / Prediction_Function /
Dealloc_Buffers with MLIR's expanded memref descriptors, called the way
src/gpu/GPUModelSerializers.cpp:21-262 calls them -- here through ctypes (dlopen + dlsym) with
hand-built descriptors -- and checked against the oracle; and the reorg serializer's flavour
(Init_Thresholds / Init_FeatureIndices, src/gpu/ReorgForestRepresentation.cpp:278-377) from
the second library.

The buffers are serialized by a restatement of the reference's scalar layouts:
array (src/include/DecisionForest.h:292-315: a complete array per tree, children of slot i at
2i+1 / 2i+2, leaf = feature index -1 with its value in the threshold, unused slots 0 / -1) and
sparse (:595-629: level order, child index = left child, right child = left + 1); the reorg
buffers interleave the trees' complete arrays (slot s of tree t at s * trees + t,
src/gpu/ReorgForestRepresentation.cpp:186-211, 258-276)."""
import ctypes
import os

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import assert_predictions_close, small_config

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
MODULE = os.path.join(ROOT, "treebeard_b200", "lib", "libtbk_module.so")
MODULE_REORG = os.path.join(ROOT, "treebeard_b200", "lib", "libtbk_module_reorg.so")
I64, I32, VP = ctypes.c_int64, ctypes.c_int32, ctypes.c_void_p


class Memref1(ctypes.Structure):
    _fields_ = [("bufferPtr", VP), ("alignedPtr", VP), ("offset", I64), ("lengths", I64 * 1), ("strides", I64 * 1)]


class Config(ctypes.Structure):
    _fields_ = [("batch_size", I32), ("row_size", I32), ("sparse", I32), ("feature_index_width", I32),
                ("child_index_width", I32), ("tile_shape_width", I32), ("num_classes", I32), ("transform", I32),
                ("return_width", I32), ("device", I32), ("num_trees", I32), ("reserved", I32),
                ("initial_value", ctypes.c_double)]


NAMES = ["Prediction_Function", "Init_Model", "Init_Offsets", "Init_Lengths", "Init_ClassIds", "Dealloc_Buffers",
         "GetBatchSize", "GetRowSize", "GetInputTypeBitWidth", "GetReturnTypeBitWidth", "TBK_Module_Configure",
         "TBK_Module_LastError"]


def load():
    lib = ctypes.CDLL(MODULE)
    m1 = [VP, VP, I64, I64, I64]
    lib.Init_Lengths.argtypes, lib.Init_Lengths.restype = m1, Memref1
    lib.Init_Offsets.argtypes, lib.Init_Offsets.restype = m1, Memref1
    lib.Init_ClassIds.argtypes, lib.Init_ClassIds.restype = m1, Memref1
    lib.Init_Model.argtypes, lib.Init_Model.restype = m1 * 4, Memref1
    lib.Prediction_Function.argtypes = [VP, VP, I64, I64, I64, I64, I64] + m1 * 5
    lib.Prediction_Function.restype = Memref1
    lib.Dealloc_Buffers.argtypes, lib.Dealloc_Buffers.restype = m1 * 3, I32
    lib.TBK_Module_Configure.argtypes = [ctypes.POINTER(Config)]
    lib.TBK_Module_LastError.restype = ctypes.c_char_p
    return lib


def desc(a):
    """The five arguments of a rank-1 memref over a contiguous numpy array."""
    return [a.ctypes.data, a.ctypes.data, 0, len(a), 1]


def serialize(forest, sparse, index_dtype):
    """(thresholds, feature indices, tile-shape ids, child indices, offsets, lengths) in the
    reference's scalar array / sparse layout."""
    thr, feat, child, offsets, lengths = [], [], [], [], []
    for t in range(forest.num_trees):
        a, b = int(forest.tree_off[t]), int(forest.tree_off[t + 1])
        L, R, F, V = forest.left[a:b], forest.right[a:b], forest.feat[a:b], forest.thr[a:b]
        if sparse:
            order, nxt = [0], 0                      # level order from the root
            while nxt < len(order):
                n = order[nxt]; nxt += 1
                if L[n] >= 0:
                    order += [int(L[n]), int(R[n])]
            where = {n: i for i, n in enumerate(order)}
            tt = np.array([V[n] for n in order], np.float32)
            ff = np.array([F[n] if L[n] >= 0 else -1 for n in order], index_dtype)
            cc = np.array([where[int(L[n])] if L[n] >= 0 else -1 for n in order], index_dtype)
        else:
            depth = 1
            stack = [(0, 1)]
            while stack:
                n, d = stack.pop(); depth = max(depth, d)
                if L[n] >= 0:
                    stack += [(int(L[n]), d + 1), (int(R[n]), d + 1)]
            tt = np.zeros(2 ** depth - 1, np.float32)
            ff = np.full(2 ** depth - 1, -1, index_dtype)
            cc = np.zeros(0, index_dtype)
            stack = [(0, 0)]
            while stack:
                n, slot = stack.pop()
                tt[slot] = V[n]
                if L[n] >= 0:
                    ff[slot] = F[n]
                    stack += [(int(L[n]), 2 * slot + 1), (int(R[n]), 2 * slot + 2)]
        offsets.append(sum(lengths)); lengths.append(len(tt))
        thr.append(tt); feat.append(ff); child.append(cc)
    cat = np.concatenate
    shapes = np.zeros(sum(lengths), np.int16)
    return (cat(thr), cat(feat), shapes, cat(child) if sparse else np.zeros(1, index_dtype),
            np.array(offsets, np.int64), np.array(lengths, np.int64))


def test_module_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(MODULE)
    header = open(os.path.join(ROOT, "include", "tbk_module.h")).read()
    for name in NAMES:
        assert name + "(" in header
        assert getattr(lib, name) is not None
    lib = load()
    bad = Config(0, 8, 0, 16, 16, 16, 0, 0, 32, 0, 0, 0, 0.0)
    assert lib.TBK_Module_Configure(ctypes.byref(bad)) != 0 and b"positive" in lib.TBK_Module_LastError()
    ok = Config(64, 8, 0, 16, 16, 16, 0, 0, 32, 0, 0, 0, 0.5)
    assert lib.TBK_Module_Configure(ctypes.byref(ok)) == 0
    assert (lib.GetBatchSize(), lib.GetRowSize(), lib.GetInputTypeBitWidth(), lib.GetReturnTypeBitWidth()) == (64, 8, 32, 32)


@pytest.mark.gpu
@pytest.mark.parametrize("name,sparse,index_dtype", [("c1", False, np.int16), ("c2", True, np.int16),
                                                     ("c2", False, np.int32), ("c4", True, np.int32)])
def test_module_calls_match_the_oracle(name, sparse, index_dtype):
    forest, X = small_config(name, rows=512)
    want, sums = oracle.predict(forest, X, class_sums=True)
    lib = load()
    width = 8 * np.dtype(index_dtype).itemsize
    multiclass = forest.num_classes > 0
    cfg = Config(len(X), forest.num_features, int(sparse), width, width, 16, forest.num_classes, forest.transform,
                 8 if multiclass else 32, 0, 0, 0, forest.initial_value)
    assert lib.TBK_Module_Configure(ctypes.byref(cfg)) == 0, lib.TBK_Module_LastError()
    thr, feat, shapes, child, offsets, lengths = serialize(forest, sparse, index_dtype)
    lengths_m = lib.Init_Lengths(*desc(lengths))
    offsets_m = lib.Init_Offsets(*desc(offsets))
    model_m = lib.Init_Model(*(desc(thr) + desc(feat) + desc(shapes) + desc(child)))
    assert model_m.lengths[0] == len(thr), lib.TBK_Module_LastError()
    class_ids = forest.class_id.astype(np.int8)
    class_m = lib.Init_ClassIds(*desc(class_ids)) if multiclass else Memref1(None, None, 0, (I64 * 1)(0), (I64 * 1)(1))

    def m(x):
        return [x.bufferPtr, x.alignedPtr, x.offset, x.lengths[0], x.strides[0]]
    out = np.zeros(len(X), np.int8 if multiclass else np.float32)
    for _ in range(2):                               # a second call reuses the uploaded forest
        res = lib.Prediction_Function(X.ctypes.data, X.ctypes.data, 0, X.shape[0], X.shape[1], X.shape[1], 1,
                                      *(desc(out) + m(model_m) + m(offsets_m) + m(lengths_m) + m(class_m)))
        assert lib.TBK_Module_LastError() == b"", lib.TBK_Module_LastError()
        assert res.alignedPtr == out.ctypes.data and res.lengths[0] == len(out)
        assert_predictions_close(out.astype(np.float32), want, forest, sums)
    assert lib.Dealloc_Buffers(*(m(model_m) + m(offsets_m) + m(lengths_m))) == 0


REORG_NAMES = ["Prediction_Function", "Init_Thresholds", "Init_FeatureIndices", "Init_ClassIds", "Dealloc_Buffers",
               "GetBatchSize", "GetRowSize", "GetInputTypeBitWidth", "GetReturnTypeBitWidth", "TBK_Module_Configure",
               "TBK_Module_LastError"]


def load_reorg():
    lib = ctypes.CDLL(MODULE_REORG)
    m1 = [VP, VP, I64, I64, I64]
    lib.Init_Thresholds.argtypes, lib.Init_Thresholds.restype = m1, Memref1
    lib.Init_FeatureIndices.argtypes, lib.Init_FeatureIndices.restype = m1, Memref1
    lib.Init_ClassIds.argtypes, lib.Init_ClassIds.restype = m1, Memref1
    lib.Prediction_Function.argtypes = [VP, VP, I64, I64, I64, I64, I64] + m1 * 4
    lib.Prediction_Function.restype = Memref1
    lib.Dealloc_Buffers.restype = I32
    lib.TBK_Module_Configure.argtypes = [ctypes.POINTER(Config)]
    lib.TBK_Module_LastError.restype = ctypes.c_char_p
    return lib


def serialize_reorg(forest, index_dtype):
    """(thresholds, feature indices): the trees' complete arrays, all of the deepest tree's
    size, interleaved tree by tree."""
    thr, feat, _, _, _, lengths = serialize(forest, False, index_dtype)
    T, slots = forest.num_trees, int(lengths.max())
    tt = np.full(slots * T, -1e6, np.float32)
    ff = np.full(slots * T, -1, index_dtype)
    at = 0
    for t in range(T):
        n = int(lengths[t])
        tt[t:n * T:T] = thr[at:at + n]
        ff[t:n * T:T] = feat[at:at + n]
        at += n
    return tt, ff


def test_reorg_module_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(MODULE_REORG)
    header = open(os.path.join(ROOT, "include", "tbk_module.h")).read()
    for name in REORG_NAMES:
        assert name + "(" in header
        assert getattr(lib, name) is not None
    for name in ("Init_Model", "Init_Offsets", "Init_Lengths"):
        assert not hasattr(lib, name)
    lib = load_reorg()
    cfg = Config(64, 8, 0, 16, 16, 16, 0, 0, 32, 0, 0, 0, 0.5)       # num_trees left at 0
    assert lib.TBK_Module_Configure(ctypes.byref(cfg)) == 0
    thr, feat = np.zeros(7, np.float32), np.full(7, -1, np.int16)
    lib.Init_Thresholds(*desc(thr)); lib.Init_FeatureIndices(*desc(feat))
    X, out = np.zeros((64, 8), np.float32), np.zeros(64, np.float32)
    z = [None, None, 0, 0, 1]
    lib.Prediction_Function(X.ctypes.data, X.ctypes.data, 0, 64, 8, 8, 1, *(desc(out) + desc(thr) + desc(feat) + z))
    assert b"num_trees" in lib.TBK_Module_LastError()              # refused on the host, nothing launched


@pytest.mark.gpu
@pytest.mark.parametrize("name,index_dtype", [("c1", np.int8), ("c2", np.int16), ("c4", np.int32)])
def test_reorg_module_calls_match_the_oracle(name, index_dtype):
    forest, X = small_config(name, rows=512)
    want, sums = oracle.predict(forest, X, class_sums=True)
    lib = load_reorg()
    width = 8 * np.dtype(index_dtype).itemsize
    multiclass = forest.num_classes > 0
    cfg = Config(len(X), forest.num_features, 0, width, 16, 16, forest.num_classes, forest.transform,
                 8 if multiclass else 32, 0, forest.num_trees, 0, forest.initial_value)
    assert lib.TBK_Module_Configure(ctypes.byref(cfg)) == 0, lib.TBK_Module_LastError()
    thr, feat = serialize_reorg(forest, index_dtype)
    thr_m = lib.Init_Thresholds(*desc(thr))
    feat_m = lib.Init_FeatureIndices(*desc(feat))
    assert thr_m.lengths[0] == len(thr) and feat_m.lengths[0] == len(feat), lib.TBK_Module_LastError()
    class_ids = forest.class_id.astype(np.int8)
    class_m = lib.Init_ClassIds(*desc(class_ids)) if multiclass else Memref1(None, None, 0, (I64 * 1)(0), (I64 * 1)(1))

    def m(x):
        return [x.bufferPtr, x.alignedPtr, x.offset, x.lengths[0], x.strides[0]]
    out = np.zeros(len(X), np.int8 if multiclass else np.float32)
    for _ in range(2):
        res = lib.Prediction_Function(X.ctypes.data, X.ctypes.data, 0, X.shape[0], X.shape[1], X.shape[1], 1,
                                      *(desc(out) + m(thr_m) + m(feat_m) + m(class_m)))
        assert lib.TBK_Module_LastError() == b"", lib.TBK_Module_LastError()
        assert res.alignedPtr == out.ctypes.data and res.lengths[0] == len(out)
        assert_predictions_close(out.astype(np.float32), want, forest, sums)
    lib.Dealloc_Buffers.argtypes = [VP, VP, I64, I64, I64] * (3 if multiclass else 2)
    assert lib.Dealloc_Buffers(*(m(thr_m) + m(feat_m) + (m(class_m) if multiclass else []))) == 0
