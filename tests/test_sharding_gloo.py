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
    # an N that does not divide: the first N % world shards are one column wider, nothing is lost
    assert [sharded.shard_bounds(10, 3, r) for r in range(3)] == [(0, 4), (4, 7), (7, 10)]
    assert [sharded.shard_bounds(151936 + 5, 8, r)[1] - sharded.shard_bounds(151936 + 5, 8, r)[0]
            for r in range(8)] == [18993] * 5 + [18992] * 3
    assert sharded.widest_shard(10, 3) == 4
    with pytest.raises(ValueError):
        sharded.shard_bounds(10, 3, 3)
    with pytest.raises(ValueError):
        sharded.shard_bounds(0, 2, 0)
    g = np.arange(2 * 3 * 4).reshape(2, 3, 4)
    whole = sharded.assemble(g)
    assert whole.shape == (3, 8) and list(whole[1]) == [4, 5, 6, 7, 16, 17, 18, 19]
    assert torch.equal(sharded.assemble(torch.from_numpy(g)), torch.from_numpy(whole))
    ragged = sharded.assemble(g, n=7)   # shards of 4 and 3 columns in windows of 4
    assert ragged.shape == (3, 7) and list(ragged[1]) == [4, 5, 6, 7, 16, 17, 18]
    assert torch.equal(sharded.assemble(torch.from_numpy(g), n=7), torch.from_numpy(ragged))


def test_ragged_column_shards_cover_the_node_once():
    """Vocabulary tail: N = 259 over 4 shards (65, 65, 65, 64 columns) reassembles exactly."""
    from oracle import nbits_oracle as o

    full = syn.config5(m=2, bits=4, n=259)
    world = 4
    width = sharded.widest_shard(full.n, world)
    gathered = np.zeros((world, full.m, width), dtype=np.float32)
    covered = []
    for rank in range(world):
        shard = syn.shard_columns(full, world, rank)
        lo, hi = sharded.shard_bounds(full.n, world, rank)
        assert shard.meta["col_offset"] == lo and shard.n == hi - lo
        covered += list(range(lo, hi))
        gathered[rank, :, :shard.n] = o.matmul_f64(full.a, shard.b, shard.scales, shard.zero_points, shard.bias,
                                                   shard.n, shard.k, shard.bits, shard.block_size, threads=1)
    assert covered == list(range(full.n))
    expect = o.matmul_f64(full.a, full.b, full.scales, full.zero_points, full.bias, full.n, full.k, full.bits,
                          full.block_size, threads=1).astype(np.float32)
    assert np.array_equal(sharded.assemble(gathered, n=full.n), expect)


def _layout_worker(rank: int, world: int, port: int, results):
    """The host logic of the peer gather on CPU ranks: every rank derives the buffer layout and its
    pointer tables from the C++ helper, the 'handles' (here: fake base addresses) travel over the
    process group like the real ones, and the ranks' views of the layout must agree."""
    import ctypes

    from onnx_light_cpu_b200._register import _host_lib

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lib = _host_lib()
        m_max, n_shard, slots = 8, 16032, 2
        out = (ctypes.c_int64 * 4)()
        assert lib.olc_peer_gather_layout(world, rank, m_max, n_shard, slots, out) == 0
        slot_floats, flags_offset, total, window = list(out)
        assert slot_floats == world * m_max * n_shard and window == m_max * n_shard * 4
        assert flags_offset % 256 == 0 and flags_offset >= slots * slot_floats * 4
        assert total == flags_offset + slots * 256
        # each rank "allocates" a buffer at a fake address and tells the others
        base = 0x7000_0000_0000 + rank * 0x1_0000_0000
        bases = [None] * world
        dist.all_gather_object(bases, base)
        tables = {}
        for slot in range(slots):
            y = (ctypes.c_uint64 * world)()
            flags = (ctypes.c_uint64 * world)()
            assert lib.olc_peer_gather_tables(world, rank, m_max, n_shard, slots, slot,
                                              (ctypes.c_uint64 * world)(*bases), y, flags) == 0
            tables[slot] = (list(y), list(flags))
        everyone = [None] * world
        dist.all_gather_object(everyone, tables)
        ok = True
        for slot in range(slots):
            for target in range(world):
                # in rank `target`'s buffer the writers' windows tile the slot without overlap
                starts = sorted(everyone[writer][slot][0][target] - bases[target] for writer in range(world))
                ok = ok and starts == [(slot * world + w) * window for w in range(world)]
                # and every writer addresses the same flag array there
                ok = ok and len({everyone[writer][slot][1][target] for writer in range(world)}) == 1
                ok = ok and everyone[0][slot][1][target] - bases[target] == flags_offset + slot * 256
        # bad arguments are refused, not computed with
        ok = ok and lib.olc_peer_gather_layout(9, 0, 1, 1, 1, out) == 1
        ok = ok and lib.olc_peer_gather_layout(world, world, 1, 1, 1, out) == 1
        ok = ok and lib.olc_peer_gather_tables(world, rank, m_max, n_shard, slots, slots,
                                               (ctypes.c_uint64 * world)(*bases), y, flags) == 1
        results[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_peer_gather_layout_agrees_between_ranks():
    world = 2
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_layout_worker, args=(world, _free_port(), results), nprocs=world, join=True)
    assert dict(results) == {0: True, 1: True}
