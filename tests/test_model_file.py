"""Compiled-model files (binary forest + bound options) and their globals JSON: the
counterpart of the reference's ahead-of-time .so + globals JSON pair
(src/runtime/runtime.cpp:35-54, src/python/treebeard.py:314-316, 385-389)."""
import json
import os

import numpy as np
import pytest

from oracle import oracle
from tests.helpers import assert_predictions_close, small_config
from treebeard_b200 import synth, treebeard


def _write(tmp_path, name="c2", trees=48, batch=64, **kw):
    forest, X = small_config(name, rows=batch, trees=trees)
    model = str(tmp_path / "m.json")
    synth.save_xgboost_json(forest, model)
    options = treebeard.CompilerOptions(batch, kw.get("tile", 1))
    if forest.num_classes:
        options.SetReturnTypeWidth(8)
        options.SetReturnTypeIsFloatType(False)
    out, glob = str(tmp_path / "m.tbmodel"), str(tmp_path / "m.globals.json")
    treebeard.GenerateLLVMIRForXGBoostModel(model, out, glob, options)
    return forest, X, out, glob


def test_model_file_round_trip_on_host(tmp_path):
    forest, X, out, glob = _write(tmp_path)
    back = treebeard.LoadForest(out, "compiled_model")
    for name in ("tree_off", "left", "right", "thr", "class_id"):
        assert np.array_equal(getattr(back, name), getattr(forest, name)), name
    split = forest.left >= 0
    assert np.array_equal(back.feat[split], forest.feat[split])
    assert back.transform == forest.transform and back.num_features == forest.num_features
    assert back.initial_value == pytest.approx(forest.initial_value)
    assert np.array_equal(oracle.predict(back, X), oracle.predict(forest, X))
    g = json.load(open(glob))
    entry, = g["TileSizeEntries"]
    assert entry == {"TileSize": 1, "ThresholdBitWidth": 32, "FeatureIndexBitWidth": 16}
    assert g["BatchSize"] == 64 and g["RowSize"] == forest.num_features
    assert g["NumberOfTrees"] == forest.num_trees and g["Representation"] in ("gpu_array", "gpu_sparse", "gpu_auto")


def test_model_file_rejects_damage(tmp_path):
    _, _, out, _ = _write(tmp_path)
    blob = open(out, "rb").read()
    cases = {
        "bad magic": b"NOTAFILE" + blob[8:],
        "truncated": blob[:1000],                         # inside the forest arrays
        "flipped byte": blob[:200] + bytes([blob[200] ^ 0x40]) + blob[201:],
        "trailing bytes": blob + b"\0" * 8,
        "empty": b"",
    }
    for what, data in cases.items():
        path = str(tmp_path / "bad.tbmodel")
        open(path, "wb").write(data)
        with pytest.raises(treebeard.TreebeardRuntimeError):
            treebeard.LoadForest(path, "compiled_model")
        with pytest.raises(treebeard.TreebeardRuntimeError):
            treebeard.TreebeardInferenceRunner.FromSOFile(path, "")
    with pytest.raises(treebeard.TreebeardRuntimeError):
        treebeard.TreebeardInferenceRunner.FromSOFile(str(tmp_path / "missing.tbmodel"), "")


def test_context_dump_writes_both_files(tmp_path):
    forest, _ = small_config("c1", rows=32, trees=20)
    model = str(tmp_path / "m.json")
    synth.save_xgboost_json(forest, model)
    glob = str(tmp_path / "ctx.globals.json")
    ctx = treebeard.TreebeardContext(model, glob, treebeard.CompilerOptions(32, 2),
                                     treebeard.GPUAutoScheduleOptions.Construct(64, 1, 4))
    ctx.SetRepresentationType("gpu_reorg")
    out = str(tmp_path / "ctx.tbmodel")
    ctx.DumpLLVMIR(out)
    assert os.path.getsize(out) > 0
    g = json.load(open(glob))
    assert g["Representation"] == "gpu_reorg" and g["TileSizeEntries"][0]["TileSize"] == 2
    assert g["GPUSchedule"]["Pinned"] is True and g["GPUSchedule"]["NumRowsPerTB"] == 64
    assert g["GPUSchedule"]["NumTreeThreads"] == 4


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["c1", "c2", "c4"])
def test_runner_from_model_file_matches_direct_runner(name, tmp_path):
    forest, X, out, glob = _write(tmp_path, name=name, trees=52, batch=256)
    runner = treebeard.TreebeardInferenceRunner.FromSOFile(out, glob)
    kind = np.int8 if forest.num_classes else np.float32
    got = runner.RunInference(X, kind)
    want, sums = oracle.predict(forest, X, class_sums=True)
    assert_predictions_close(got, want, forest, sums)
    # the globals JSON wins over the binary: another batch size and representation
    g = json.load(open(glob))
    g["BatchSize"], g["Representation"] = 128, "gpu_sparse"
    json.dump(g, open(glob, "w"))
    runner2 = treebeard.TreebeardInferenceRunner.FromSOFile(out, glob)
    assert runner2.batchSize == 128
    got2 = runner2.RunInference(X[:128], kind)
    assert_predictions_close(got2, want[:128], forest, sums[:128] if sums is not None else None)


# ---- the packed image that a compiled-model file caches


@pytest.mark.parametrize("name,layout", [("c2", dict(representation="sparse", tile_size=2)),
                                         ("c4", dict(representation="array")),
                                         ("c3", dict(representation="auto")),
                                         ("c2", dict(representation="auto")),
                                         ("c4", dict(representation="auto", feature_bits=16)),
                                         ("c5", dict(representation="auto"))])
def test_packed_image_survives_serialisation(name, layout):
    """Host only: pack, serialise, read back, serialise again -- same bytes; a changed layout
    request or shared-memory limit does not match; damaged bytes are refused."""
    from treebeard_b200 import kernels
    forest, _ = small_config(name)
    image = kernels.PackedImage.pack(forest, **layout)
    data = image.to_bytes()
    again = kernels.PackedImage.from_bytes(data)
    assert again.to_bytes() == data
    assert again.matches(**layout)
    assert not again.matches(**dict(layout, tile_size=3))
    assert not again.matches(smem_limit=100 * 1024, **layout)
    for bad in (data[:-9], data[:100] + bytes([data[100] ^ 1]) + data[101:], b"", data + b"\0"):
        with pytest.raises(kernels.TbkError):
            kernels.PackedImage.from_bytes(bad)


def test_model_file_with_damaged_image_section_still_loads(tmp_path):
    """The forest arrays have their own checksum: a packed-image section that is cut short or
    altered costs only the shortcut (the loader packs again), never the model."""
    forest, X, out, _ = _write(tmp_path)
    blob = open(out, "rb").read()
    bare = treebeard.LoadForest(out, "compiled_model")
    marker = blob.index(b"TBB2SEC1")
    assert marker > 0 and len(blob) - marker > 1000       # the file does carry an image
    for what, data in {"cut short": blob[: marker + 500], "no section": blob[:marker],
                       "altered": blob[: marker + 300] + bytes([blob[marker + 300] ^ 0x10]) + blob[marker + 301:]}.items():
        path = str(tmp_path / "cut.tbmodel")
        open(path, "wb").write(data)
        back = treebeard.LoadForest(path, "compiled_model")
        assert np.array_equal(back.thr, bare.thr) and np.array_equal(back.left, bare.left), what


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["c2", "c3", "c5"])
def test_runner_from_model_file_uses_the_packed_image(name, tmp_path):
    trees = {"c2": 52, "c3": 40, "c5": 12}[name]
    forest, X, out, glob = _write(tmp_path, name=name, trees=trees, batch=256)
    g = json.load(open(glob))
    # ask for another representation than the file was written for (the process default:
    # "gpu_auto" unless the sparse switch was touched): the forest is packed again
    g["Representation"] = "gpu_sparse" if g["Representation"] == "gpu_auto" else "gpu_auto"
    json.dump(g, open(glob, "w"))
    want = oracle.predict(forest, X)
    runner = treebeard.TreebeardInferenceRunner.FromSOFile(out, glob)
    assert not runner.used_packed_image()
    assert_predictions_close(runner.RunInference(X), want)
    # written for the same request: the image is uploaded as it is
    model = str(tmp_path / "m.json")
    ctx = treebeard.TreebeardContext(model, glob, treebeard.CompilerOptions(256, 1))
    ctx.SetRepresentationType("gpu_auto")
    out2 = str(tmp_path / "auto.tbmodel")
    ctx.DumpLLVMIR(out2)
    cached = treebeard.TreebeardInferenceRunner.FromSOFile(out2, "")
    assert cached.used_packed_image()
    assert_predictions_close(cached.RunInference(X), want)
    # an altered image is dropped, the result stays right
    blob = open(out2, "rb").read()
    k = blob.index(b"TBB2SEC1") + 4000
    open(out2, "wb").write(blob[:k] + bytes([blob[k] ^ 0x20]) + blob[k + 1:])
    fallback = treebeard.TreebeardInferenceRunner.FromSOFile(out2, "")
    assert not fallback.used_packed_image()
    assert_predictions_close(fallback.RunInference(X), want)
