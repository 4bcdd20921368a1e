"""Parity at the configurations' FULL sizes, through the C ABI.

The oracle cannot walk 10^9..10^11 (row, tree) pairs in test time, so at full size the
checks are (a) the oracle on a seeded subsample of rows against the same rows of the
full-batch GPU result -- leaf ids bit-exact, predictions within tolerance -- and (b)
size-independent properties: a batch split at an odd row gives the same predictions as the
whole batch, and the raw partial sums of two halves of the forest add up to the whole."""
import numpy as np
import pytest

from oracle import oracle
from tests.helpers import assert_predictions_close
from treebeard_b200 import synth

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")

# name, rows on the device, rows checked against the oracle, rows for the leaf-id matrix
# (the three batch sizes of the binary classifier select three different launch shapes)
FULL = [("c1", 1024, 1024, 1024), ("c2", 4096, 4096, 1024), ("c2", 65536, 65536, 2048),
        ("c2", 1048576, 65536, 2048), ("c3", 262144, 65536, 4096), ("c4", 1048576, 16384, 1024)]


@pytest.mark.parametrize("name,rows,check,leaf_rows", FULL)
def test_full_size_configuration(name, rows, check, leaf_rows):
    from treebeard_b200 import kernels
    forest, marg, _ = synth.make_config(name)
    X = synth.config_rows(name, marg, rows)
    dX = torch.from_numpy(X).cuda()
    df = kernels.DeviceForest(forest, representation="auto", batch_hint=rows)
    got = df.predict(dX)
    df.check_status()
    pick = np.sort(np.random.Generator(np.random.PCG64(7)).choice(rows, size=check, replace=False))
    want, sums = oracle.predict(forest, X[pick], class_sums=True)
    assert_predictions_close(got.cpu().numpy()[pick], want, forest, sums)
    # leaf selection, bit-exact, on a subsample (the full matrix would be rows x trees)
    sub = pick[:leaf_rows]
    _, want_ids = oracle.predict(forest, X[sub], leaf_ids=True)
    ids = df.predict_leaf_ids(torch.from_numpy(X[sub]).cuda()).cpu().numpy()
    assert np.array_equal(ids, want_ids)
    # split-batch consistency at an odd boundary
    if rows > 5000:
        k = rows // 3 + 1
        a, b = df.predict(dX[:k]), df.predict(dX[k:])
        whole = got.cpu().numpy()
        parts = torch.cat([a, b]).cpu().numpy()
        if forest.num_classes:
            assert (parts != whole).mean() < 1e-4      # only exact class-sum ties may flip
        else:
            assert_predictions_close(parts, whole)


def test_full_size_tree_shards_add_up():
    """C5's shape at a reduced forest (the full 16 000-tree forest is a benchmark run):
    partial sums of two tree shards add up to the predictions of the whole forest."""
    from treebeard_b200 import kernels
    forest, marg, _ = synth.make_config("c5", trees=512)
    rows = 65536
    X = synth.config_rows("c5", marg, rows)
    dX = torch.from_numpy(X).cuda()
    whole = kernels.DeviceForest(forest, representation="auto", batch_hint=rows)
    half = forest.num_trees // 2
    a = kernels.DeviceForest(forest.tree_slice(0, half), batch_hint=rows)
    b = kernels.DeviceForest(forest.tree_slice(half, forest.num_trees), batch_hint=rows)
    total = a.predict_partial(dX) + b.predict_partial(dX)
    got = whole.finalize(total).cpu().numpy()
    assert_predictions_close(got, whole.predict(dX).cpu().numpy())
    pick = np.arange(0, rows, 64)
    want, want_ids = oracle.predict(forest, X[pick], leaf_ids=True)
    assert_predictions_close(got[pick], want)
    ids = whole.predict_leaf_ids(torch.from_numpy(X[pick[:256]]).cuda()).cpu().numpy()
    assert np.array_equal(ids, want_ids[:256])


def test_full_size_large_forest_c5():
    """C5 with all 16 000 trees (deep-tree kernel): the oracle on a subsample of a 65 536-row
    batch -- leaf ids bit-exact for every tree, predictions within tolerance -- and the
    batch split at an odd row."""
    from treebeard_b200 import kernels
    forest, marg, _ = synth.make_config("c5")
    rows = 65536
    X = synth.config_rows("c5", marg, rows)
    dX = torch.from_numpy(X).cuda()
    df = kernels.DeviceForest(forest, representation="auto", batch_hint=rows)
    assert df.info().schedule.feature_bits == 16
    got = df.predict(dX).cpu().numpy()
    df.check_status()
    pick = np.sort(np.random.Generator(np.random.PCG64(11)).choice(rows, size=8192, replace=False))
    want = oracle.predict(forest, X[pick])
    assert_predictions_close(got[pick], want)
    _, want_ids = oracle.predict(forest, X[pick[:1024]], leaf_ids=True)
    ids = df.predict_leaf_ids(torch.from_numpy(X[pick[:1024]]).cuda()).cpu().numpy()
    assert np.array_equal(ids, want_ids)
    k = rows // 3 + 1
    parts = torch.cat([df.predict(dX[:k]), df.predict(dX[k:])]).cpu().numpy()
    assert_predictions_close(parts, got)
