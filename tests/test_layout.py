"""Forest-to-buffer lowering, checked on the host: the packed buffers are interpreted on
the CPU with the kernels' slot arithmetic and must select exactly the leaves the oracle
selects, for every representation and tile size."""
import numpy as np
import pytest

from oracle import oracle
from tests.helpers import SMALL, small_config
from treebeard_b200 import kernels, synth

REPS = [("sparse", 1), ("sparse", 2), ("sparse", 3), ("sparse", 4), ("array", 1), ("array", 2),
        ("array", 3), ("array", 4), ("reorg", 1)]


@pytest.mark.parametrize("name", list(SMALL))
@pytest.mark.parametrize("rep,ts", REPS)
def test_packed_layout_selects_oracle_leaves(name, rep, ts):
    if name == "c5" and rep == "array" and ts > 1:
        pytest.skip("array layout of deep unbalanced trees is too large by construction")
    forest, X = small_config(name, rows=200)
    _, want_ids, class_sums = oracle.predict(forest, X, leaf_ids=True, class_sums=True)
    ids, sums, info = kernels.host_layout_check(forest, X, representation=rep, tile_size=ts)
    assert np.array_equal(ids, want_ids)
    g = forest.tree_off[:-1][None, :] + want_ids
    if forest.num_classes == 0:
        want = forest.thr[g].astype(np.float64).sum(axis=1)
        assert np.allclose(sums[:, 0], want, rtol=1e-5, atol=1e-5)
    else:
        assert np.allclose(sums, class_sums - forest.initial_value, rtol=1e-5, atol=1e-5)
    if forest.num_classes == 0:
        assert info.num_groups == (forest.num_trees + 15) // 16
    else:   # every class is padded to whole groups of its own
        per_class = np.bincount(forest.class_id, minlength=forest.num_classes)
        assert info.num_groups == sum(max(1, (n + 15) // 16) for n in per_class)


@pytest.mark.parametrize("ts,shapes", [(1, 1), (2, 3), (3, 8), (4, 22)])
def test_tile_shape_count_is_the_catalan_sum(ts, shapes):
    forest, _ = small_config("c1", rows=1)
    _, _, info = kernels.host_layout_check(forest, None, representation="sparse", tile_size=ts)
    # + 1: the leaf tile's own shape
    assert info.reserved[0] == shapes + 1
    assert info.reserved[1] == (shapes + 1) << ts


def _tiny(left, right, feat, thr, F=3):
    n = len(left)
    return synth.ForestArrays(np.array([0, n], np.int64), np.array(left, np.int32),
                              np.array(right, np.int32), np.array(feat, np.int32),
                              np.array(thr, np.float32), np.zeros(1, np.int32), 0, 0, 0.0, F)


def test_hand_trees_every_outcome():
    # left-heavy chain, right-heavy chain and a balanced tree, all outcomes enumerated
    chains = [
        _tiny([1, 3, -1, 5, -1, -1, -1], [2, 4, -1, 6, -1, -1, -1], [0, 1, 0, 2, 0, 0, 0],
              [0.5, 0.5, 10, 0.5, 20, 30, 40]),
        _tiny([1, -1, 3, -1, 5, -1, -1], [2, -1, 4, -1, 6, -1, -1], [0, 0, 1, 0, 2, 0, 0],
              [0.5, 10, 0.5, 20, 0.5, 30, 40]),
        _tiny([1, 3, 5, -1, -1, -1, -1], [2, 4, 6, -1, -1, -1, -1], [0, 1, 2, 0, 0, 0, 0],
              [0.5, 0.5, 0.5, 1, 2, 3, 4]),
    ]
    X = np.array([[a, b, c] for a in (0.0, 0.5, 1.0) for b in (0.0, 0.5, 1.0) for c in (0.0, 0.5, 1.0)],
                 np.float32)
    for forest in chains:
        _, want = oracle.predict(forest, X, leaf_ids=True)
        for rep, ts in REPS:
            ids, _, _ = kernels.host_layout_check(forest, X, representation=rep, tile_size=ts)
            assert np.array_equal(ids, want), (rep, ts)


def test_single_leaf_tree_and_filler_columns():
    forest = synth.ForestArrays(np.array([0, 1, 4], np.int64), np.array([-1, 1, -1, -1], np.int32),
                                np.array([-1, 2, -1, -1], np.int32), np.array([0, 1, 0, 0], np.int32),
                                np.array([7.0, 0.0, -1.0, 1.0], np.float32), np.zeros(2, np.int32),
                                0, 0, 0.0, 2)
    X = np.array([[0, -1], [0, 0], [0, 1]], np.float32)
    for rep, ts in REPS:
        ids, sums, _ = kernels.host_layout_check(forest, X, representation=rep, tile_size=ts)
        assert ids.tolist() == [[0, 1], [0, 2], [0, 2]]
        assert sums[:, 0].tolist() == [6.0, 8.0, 8.0]


@pytest.mark.parametrize("breakage", ["one_child", "bad_child", "bad_feature", "two_parents", "nan",
                                      "neg_inf_leaf", "reorg_tiled", "tile_too_big"])
def test_malformed_forests_are_rejected(breakage):
    forest = _tiny([1, -1, -1], [2, -1, -1], [0, 0, 0], [0.5, 1, 2])
    kw = dict(representation="sparse", tile_size=1)
    if breakage == "one_child":
        forest.right[0] = -1
    elif breakage == "bad_child":
        forest.left[0] = 9
    elif breakage == "bad_feature":
        forest.feat[0] = 3
    elif breakage == "two_parents":
        forest.right[0] = 1
    elif breakage == "nan":
        forest.thr[0] = np.nan
    elif breakage == "neg_inf_leaf":
        forest.thr[1] = -np.inf
    elif breakage == "reorg_tiled":
        kw = dict(representation="reorg", tile_size=2)
    elif breakage == "tile_too_big":
        kw = dict(representation="sparse", tile_size=5)
    with pytest.raises(kernels.TbkError):
        kernels.host_layout_check(forest, None, **kw)


@pytest.mark.parametrize("name", ["c1", "c2", "c3"])
def test_sixteen_bit_key_layout_is_exact_including_ties(name):
    """Wide-row layout: rows as order-preserving 16-bit keys.  Key ties (forced here by
    copying thresholds into the rows), NaN and infinities must still select the oracle's
    leaves, because ties are decided on the exact fp32 values."""
    forest, X = small_config(name, rows=400)
    X = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(300):
        g = split[(i * 37) % len(split)]
        X[i % len(X), forest.feat[g]] = forest.thr[g]
    X[3, :] = np.nan
    X[4, 0] = np.inf
    X[5, 1] = -np.inf
    _, want = oracle.predict(forest, X, leaf_ids=True)
    ids, sums, info = kernels.host_layout_check(forest, X, representation="reorg", feature_bits=16)
    assert np.array_equal(ids, want)
    assert info.schedule.feature_bits == 16 and info.reserved[0] >= 5   # ties were exercised
    assert info.num_groups == (forest.num_trees + 31) // 32


@pytest.mark.parametrize("trees", [1, 7, 24])
def test_deep_tree_key_layout_is_exact_including_ties(trees):
    """Deep trees (9..12 levels): one complete tree per stage, rows as 16-bit keys, two
    trees per pair.  Same exactness requirement as the wide-row layout."""
    forest, X = small_config("c5", rows=300, trees=trees)
    X = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(250):
        g = split[(i * 101) % len(split)]
        X[i % len(X), forest.feat[g]] = forest.thr[g]
    for i in range(6, 40):                      # ties at roots are always reached
        g = forest.tree_off[i % trees]
        X[i, forest.feat[g]] = forest.thr[g]
    X[3, :] = np.nan
    X[4, 0] = np.inf
    X[5, 1] = -np.inf
    want_pred, want = oracle.predict(forest, X, leaf_ids=True)
    ids, sums, info = kernels.host_layout_check(forest, X, representation="reorg", feature_bits=16)
    assert np.array_equal(ids, want)
    assert info.max_depth > 8 and info.num_groups == (forest.num_trees + 1) // 2
    assert info.schedule.feature_bits == 16
    assert info.reserved[0] >= 5   # ties were exercised
    np.testing.assert_allclose(sums[:, 0] + forest.initial_value, want_pred, rtol=1e-5, atol=1e-6)


def test_sixteen_bit_keys_refuse_what_they_cannot_hold():
    # 13 levels: a whole-tree stage would need 32 KB planes
    chain = synth.generate_forest(5, 2, 13, 4, 0.3, 0.1, synth.Marginal("uniform01", 4))
    with pytest.raises(kernels.TbkError, match="deeper"):
        kernels.host_layout_check(chain, None, representation="reorg", feature_bits=16)


def test_sixteen_bit_keys_lay_multiclass_forests_out_class_by_class():
    """Every class fills whole groups of 32 columns; the host interpreter of the packed planes
    must find the oracle's leaves and per-class sums."""
    forest, X = small_config("c4", rows=300)
    want, want_ids = oracle.predict(forest, X, leaf_ids=True)
    _, sums_want = oracle.predict(forest, X, class_sums=True)
    ids, sums, info = kernels.host_layout_check(forest, X, representation="reorg", feature_bits=16)
    assert np.array_equal(ids, want_ids)
    assert np.allclose(sums, sums_want - forest.initial_value, rtol=1e-5, atol=1e-5) or \
        np.allclose(sums, sums_want, rtol=1e-5, atol=1e-5)
    per_class = np.bincount(forest.class_id, minlength=forest.num_classes)
    assert info.num_groups == sum(max(1, -(-int(n) // 32)) for n in per_class)
    # C4's features and thresholds are whole numbers: lattice features, whose whole-number rows
    # never tie although one comparison in 16 is an exact equality
    assert info.reserved[0] == 0
    # rows that are not whole numbers, hugging thresholds from both sides, infinities and NaN:
    # decided by the keys where they can, by the exact comparison otherwise -- always the oracle's leaf
    Y = X.copy()
    split = np.nonzero(forest.left >= 0)[0]
    for i in range(4000):
        g = split[(i * 37) % len(split)]
        Y[i % len(Y), forest.feat[g]] = forest.thr[g] + ((-1) ** i) * [1e-6, 1e-4, 0.25, 0.5][i % 4]
    Y[7, :] = np.nan
    Y[8, 0], Y[9, 1] = np.inf, -np.inf
    _, want_ids = oracle.predict(forest, Y, leaf_ids=True)
    ids, _, info = kernels.host_layout_check(forest, Y, representation="reorg", feature_bits=16)
    assert np.array_equal(ids, want_ids)
    assert info.reserved[0] > 0


def test_multiclass_class_without_trees_keeps_its_place():
    """Class-major groups: a class that no tree votes for still gets a (filler) group, so that
    its sum -- the initial value alone, as in the reference's generated reduction
    (src/reduction/LowerReduceOps.cpp:921-1003); the reference's header walker leaves such a
    class at 0 instead -- takes part in the arg-max."""
    forest, X = small_config("c4", rows=300, trees=52)
    forest.class_id[forest.class_id == 7] = 8          # nobody votes for class 7 any more
    want, want_ids, class_sums = oracle.predict(forest, X, leaf_ids=True, class_sums=True)
    class_sums[:, 7] = forest.initial_value
    ids, sums, info = kernels.host_layout_check(forest, X, representation="sparse")
    assert np.array_equal(ids, want_ids)
    assert np.allclose(sums, class_sums - forest.initial_value, rtol=1e-5, atol=1e-5)
    assert np.all(sums[:, 7] == 0.0)
    per_class = np.bincount(forest.class_id, minlength=forest.num_classes)
    assert info.num_groups == sum(max(1, (n + 15) // 16) for n in per_class)
