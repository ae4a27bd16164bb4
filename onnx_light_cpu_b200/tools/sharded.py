"""Column sharding of one MatMulNBits node over the GPUs of a box.

Every output column n needs only row n of B / scales / zero_points / bias and all of A, so the
weight rows are split into ``world`` contiguous ranges, A is replicated, each rank computes
``Y[:, lo:hi]`` and the shards are all-gathered. The gathered layout is ``[world, M, N/world]``;
:func:`assemble` turns it into the row-major ``[M, N]`` the operator defines.
"""

from __future__ import annotations

import numpy as np


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    if n % world != 0:
        raise ValueError(f"N={n} does not divide by the number of shards {world}")
    per = n // world
    return rank * per, (rank + 1) * per


def assemble(gathered):
    """[world, M, N/world] -> [M, N] (numpy array or torch tensor)."""
    world, m, per = gathered.shape
    if isinstance(gathered, np.ndarray):
        return np.ascontiguousarray(gathered.transpose(1, 0, 2)).reshape(m, world * per)
    return gathered.permute(1, 0, 2).reshape(m, world * per)


def gather_shards(y_shard, dist, out=None):
    """All-gathers equal-sized ``[M, N/world]`` shards into ``[world, M, N/world]``."""
    import torch

    world = dist.get_world_size()
    if out is None:
        out = torch.empty((world,) + tuple(y_shard.shape), dtype=y_shard.dtype, device=y_shard.device)
    if dist.get_backend() == "nccl":
        dist.all_gather_into_tensor(out, y_shard)
    else:
        parts = [out[i] for i in range(world)]
        dist.all_gather(parts, y_shard.contiguous())
    return out


class ShardedMatMulNBits:
    """One rank's share of a column-sharded node on its GPU (NCCL all-gather of the outputs)."""

    def __init__(self, b, scales, zero_points, bias, *, K, N, bits, block_size, dist):
        import onnx_light_cpu_b200 as pkg

        self.dist = dist
        self.world = dist.get_world_size()
        self.rank = dist.get_rank()
        lo, hi = shard_bounds(N, self.world, self.rank)
        nb = -(-K // block_size)
        self.n_full, self.n_shard = N, hi - lo
        self.weights = pkg.MatMulNBitsWeights(
            b[lo:hi], scales.reshape(N, nb)[lo:hi].reshape(-1),
            None if zero_points is None else zero_points[lo:hi],
            None if bias is None else bias[lo:hi], K=K, N=self.n_shard, bits=bits, block_size=block_size)

    def run(self, a, y_shard, y_gathered, accuracy_level=0):
        self.weights.matmul_device(a, y_shard, accuracy_level=accuracy_level)
        return gather_shards(y_shard, self.dist, y_gathered)
