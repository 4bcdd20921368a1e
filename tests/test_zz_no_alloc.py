"""The prediction entry point that allocates nothing (tbk_predict_noalloc).

It exists for hosts that may not allocate device memory while predicting: servers whose
memory is budgeted once at start-up, latency-critical loops that cannot risk the device
synchronisation an allocation can bring, runtimes that forbid allocations outside their own
pool.  Its tree-chunk partial sums live in a fixed array inside the library instead of a
cudaMalloc'ed buffer, so its results must equal tbk_predict's -- also on a second call,
when the array still holds the first call's partial sums.

This file sorts last on purpose: if it fails, a run that stops at the first failure has
already run every other test."""
import ctypes

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import assert_predictions_close, small_config

pytestmark = pytest.mark.gpu

torch = pytest.importorskip("torch")


def _noalloc(df, rows, int8=False):
    from treebeard_b200 import kernels
    out = torch.empty(rows.shape[0], device=rows.device, dtype=torch.int8 if int8 else torch.float32)
    rc = kernels.lib().tbk_predict_noalloc(df._h, rows.data_ptr(), rows.shape[0], rows.stride(0),
                                           out.data_ptr(), 1 if int8 else 0,
                                           torch.cuda.current_stream().cuda_stream)
    if rc != 0:
        raise kernels.TbkError(rc, kernels.lib().tbk_last_error().decode())
    return out


def test_noalloc_matches_predict_on_two_calls_in_a_row():
    from treebeard_b200 import kernels
    forest, X = small_config("c2", rows=4096)
    # several tree chunks, so that partial sums really pass through the scratch array
    df = kernels.DeviceForest(forest, representation="sparse", tree_chunks=4, batch_hint=len(X))
    first_rows = torch.from_numpy(X).cuda()
    second_rows = torch.from_numpy(np.ascontiguousarray(X[::-1][:1000])).cuda()   # other rows, other size
    for rows in (first_rows, second_rows):
        want = df.predict(rows)
        got = _noalloc(df, rows)
        torch.cuda.synchronize()
        df.check_status()
        # same kernels, same tree-chunk order: the tolerance of the parity tests is ample
        assert_predictions_close(got.cpu().numpy(), want.cpu().numpy())
        assert_predictions_close(got.cpu().numpy(), oracle.predict(forest, rows.cpu().numpy()))


def test_noalloc_multiclass_and_limits():
    from treebeard_b200 import kernels
    forest, X = small_config("c4", rows=2048)
    df = kernels.DeviceForest(forest, representation="sparse", tree_chunks=3, batch_hint=len(X))
    rows = torch.from_numpy(X).cuda()
    want = df.predict(rows, int8=True)
    got = _noalloc(df, rows, int8=True)
    assert torch.equal(got, want)
    # 26 outputs x 3 chunks x rows must fit 2 Mi floats: 40000 rows do not
    big = torch.zeros((40000, forest.num_features), device="cuda")
    with pytest.raises(kernels.TbkError, match="fixed scratch"):
        _noalloc(df, big)
    wide, Xw = small_config("c3", rows=64)
    keys = kernels.DeviceForest(wide, representation="auto")
    with pytest.raises(kernels.TbkError, match="16-bit key"):
        _noalloc(keys, torch.from_numpy(Xw).cuda())


@pytest.mark.parametrize("classes", [2, 3])
def test_noalloc_large_multiclass_batch_with_the_default_schedule(classes):
    """A batch large enough for tbk_predict to keep class sums in registers (no class table in
    shared memory): the entry point that does not allocate always writes partial sums, so its
    launch plan must keep the table.  Same class ids as tbk_predict, twice in a row."""
    from treebeard_b200 import kernels, synth
    marg = synth.Marginal("int16", 16)
    forest = synth.generate_forest(4321 + classes, 8 * classes, 6, 16, 0.1, 0.1, marg,
                                   transform=synth.SOFTMAX, num_classes=classes)
    rng = np.random.Generator(np.random.PCG64(99))
    X = marg.sample_rows(rng, 320 * 1024)             # > 2 x 148 SMs x 32 warps x 32 rows
    df = kernels.DeviceForest(forest, representation="sparse", batch_hint=len(X))
    rows = torch.from_numpy(X).cuda()
    want = df.predict(rows, int8=True)
    for _ in range(2):
        got = _noalloc(df, rows, int8=True)
        torch.cuda.synchronize()
        df.check_status()
        assert torch.equal(got, want)
    sample = slice(0, 2048)
    ref, sums = oracle.predict(forest, X[sample], class_sums=True)
    assert_predictions_close(got[sample].cpu().numpy(), ref, forest, sums)
