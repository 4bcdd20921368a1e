"""Multi-GPU plumbing: one process per GPU, torch.distributed for the exchange.

Row sharding needs no collective: rank r predicts rows [r*N/G, (r+1)*N/G) against a
full replica of the forest.  Tree sharding gives rank r trees [r*T/G, (r+1)*T/G) and
all rows; the per-row partial sums (no initial value, no transformation) are summed
onto one rank with a single reduce (NCCL over NVLink on GPUs, gloo on CPU tensors), and
that rank adds the initial value and applies the transformation."""
from __future__ import annotations


def row_range(n_rows: int, rank: int, world: int, multiple: int = 32):
    """Contiguous row range of a rank; boundaries are multiples of ``multiple`` (the
    kernels' row-tile width) except the last."""
    per = -(-n_rows // world)
    per = -(-per // multiple) * multiple
    lo = min(n_rows, rank * per)
    return lo, min(n_rows, lo + per)


def tree_range(num_trees: int, rank: int, world: int):
    """Even split of the trees (the remainder goes to the first ranks)."""
    base, extra = divmod(num_trees, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def tree_shard(forest, rank: int, world: int):
    lo, hi = tree_range(forest.num_trees, rank, world)
    return forest.tree_slice(lo, hi)


def reduce_partials(partial, dst: int = 0, group=None):
    """Sums the per-row partials of all tree shards onto rank ``dst`` (in place)."""
    import torch.distributed as dist
    dist.reduce(partial, dst=dst, op=dist.ReduceOp.SUM, group=group)
    return partial


class TreeShardedForest:
    """A forest whose trees are partitioned across the ranks of a process group."""

    def __init__(self, forest, device: int, group=None, **schedule):
        import torch.distributed as dist
        from . import kernels
        self.group = group
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.num_classes = int(forest.num_classes)
        self.local = kernels.DeviceForest(tree_shard(forest, self.rank, self.world), device=device,
                                          **schedule)

    def predict(self, rows, dst: int = 0, int8: bool = False):
        """Every rank passes the same rows; rank ``dst`` gets the predictions, the
        others None."""
        partial = self.local.predict_partial(rows)
        reduce_partials(partial, dst, self.group)
        if self.rank == dst:
            return self.local.finalize(partial, int8=int8)
        return None
