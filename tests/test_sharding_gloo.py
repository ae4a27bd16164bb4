"""Host logic of the column-sharded node with two CPU ranks over gloo: shard slicing, the
gathered layout and its reassembly. The per-shard product is computed by the CPU checker here
(no GPU in this test); the GPU kernels are covered shard by shard in test_gpu_parity.py."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from onnx_light_cpu_b200.tools import sharded
from onnx_light_cpu_b200.tools import synthetic as syn


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, results):
    from oracle import nbits_oracle as o

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = syn.config5(m=3, bits=4, n=256)   # lm-head geometry at reduced N
        shard = syn.shard_columns(full, world, rank)
        lo, hi = sharded.shard_bounds(full.n, world, rank)
        assert shard.meta["col_offset"] == lo and shard.n == hi - lo
        a = torch.from_numpy(full.a.copy())
        dist.broadcast(a, src=0)                 # A is replicated
        y = o.matmul_f64(a.numpy(), shard.b, shard.scales, shard.zero_points, shard.bias, shard.n, shard.k,
                         shard.bits, shard.block_size, threads=1).astype(np.float32)
        gathered = sharded.gather_shards(torch.from_numpy(y), dist)
        assert tuple(gathered.shape) == (world, full.m, full.n // world)
        whole = sharded.assemble(gathered).numpy()
        expect = o.matmul_f64(full.a, full.b, full.scales, full.zero_points, full.bias, full.n, full.k, full.bits,
                              full.block_size, threads=1).astype(np.float32)
        results[rank] = bool(np.array_equal(whole, expect))
    finally:
        dist.destroy_process_group()


def test_two_rank_column_shards_reassemble_to_the_full_product():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}


def test_shard_helpers():
    assert sharded.shard_bounds(128256, 8, 3) == (48096, 64128)
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 3, 0)
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    whole = sharded.assemble(g)
    assert whole.shape == (3, 8) and list(whole[1]) == [4, 5, 6, 7, 16, 17, 18, 19]
    assert torch.equal(sharded.assemble(torch.from_numpy(g)), torch.from_numpy(whole))
