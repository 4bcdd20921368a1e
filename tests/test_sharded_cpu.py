"""World-size-2 tests of the multi-GPU plumbing on CPU (gloo): row ranges, tree shards and
the reduce of per-row partial sums.  The per-shard numbers come from the CPU oracle (the
checker); what is under test is the sharding arithmetic and the exchange."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle
from tests.helpers import small_config
from treebeard_b200 import sharded


def test_row_ranges_cover_the_batch_once():
    for n in (1, 31, 32, 1000, 262144, 4194304 + 5):
        for world in (1, 2, 4, 8):
            spans = [sharded.row_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
                assert a1 == b0 and a0 <= a1
            assert all(lo % 32 == 0 for lo, _ in spans if lo < n)


def test_tree_ranges_are_even():
    for T in (1, 7, 100, 16000):
        for world in (1, 2, 4, 8):
            spans = [sharded.tree_range(T, r, world) for r in range(world)]
            sizes = [hi - lo for lo, hi in spans]
            assert sum(sizes) == T and max(sizes) - min(sizes) <= 1
            assert spans[0][0] == 0 and spans[-1][1] == T


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, name, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        forest, X = small_config(name, rows=300)
        shard = sharded.tree_shard(forest, rank, world)
        # partial sums of this shard: leaf values of its trees, no initial value
        _, ids = oracle.predict(shard, X, leaf_ids=True)
        vals = shard.thr[shard.tree_off[:-1][None, :] + ids]
        W = max(1, forest.num_classes)
        part = np.zeros((len(X), W), np.float32)
        for c in range(W):
            cols = (shard.class_id == c) if forest.num_classes else slice(None)
            part[:, c] = vals[:, cols].sum(axis=1)
        t = torch.from_numpy(part)
        sharded.reduce_partials(t, dst=0)
        # row sharding: each rank predicts its own range, nothing is exchanged
        lo, hi = sharded.row_range(len(X), rank, world)
        mine = oracle.predict(forest, X[lo:hi]) if hi > lo else np.zeros(0, np.float32)
        np.save(os.path.join(out_dir, f"rows_{rank}.npy"), mine)
        if rank == 0:
            np.save(os.path.join(out_dir, "reduced.npy"), t.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("name", ["c2", "c4"])
def test_tree_sharded_reduce_and_row_sharding_world2(name, tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), name, str(tmp_path)), nprocs=world, join=True)
    forest, X = small_config(name, rows=300)
    want, sums = oracle.predict(forest, X, class_sums=True)
    reduced = np.load(tmp_path / "reduced.npy")
    if forest.num_classes:
        assert np.allclose(reduced + forest.initial_value, sums, rtol=1e-5, atol=1e-5)
    else:
        raw = reduced[:, 0].astype(np.float64) + forest.initial_value
        assert np.allclose(1.0 / (1.0 + np.exp(-raw)), want, rtol=1e-5, atol=1e-6)
    stitched = np.concatenate([np.load(tmp_path / f"rows_{r}.npy") for r in range(world)])
    assert np.array_equal(stitched, want)
