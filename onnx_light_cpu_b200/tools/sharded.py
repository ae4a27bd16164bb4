"""Column sharding of one MatMulNBits node over the GPUs of a box.

Every output column n needs only row n of B / scales / zero_points / bias and all of A, so the
weight rows are split into ``world`` contiguous ranges, A is replicated, each rank computes
``Y[:, lo:hi]`` and the shards are gathered: either by an all-gather behind the kernel
(:class:`ShardedMatMulNBits`) or by the kernel itself, which stores its columns into every rank's
result through peer-mapped memory (:class:`PeerGather`). The gathered layout is
``[world, M, N/world]``; :func:`assemble` turns it into the row-major ``[M, N]`` the operator
defines.
"""

from __future__ import annotations

import numpy as np


def shard_bounds(n: int, world: int, rank: int) -> tuple[int, int]:
    """Columns [lo, hi) of rank ``rank``. N need not divide by ``world``: the first ``N % world``
    ranks take one column more (the C++ helper ``ShardBounds`` is the implementation)."""
    import ctypes

    from .._register import _host_lib, _raise_last

    lo, hi = ctypes.c_int64(), ctypes.c_int64()
    code = _host_lib().olc_shard_bounds(n, world, rank, ctypes.byref(lo), ctypes.byref(hi))
    if code != 0:
        _raise_last(code)
    return lo.value, hi.value


def assemble(gathered, n: int | None = None):
    """[world, M, width] -> [M, N] (numpy array or torch tensor). ``n``: the node's N when it does
    not divide by the number of shards: ``width`` is then the widest shard and rank r's valid
    columns are the first ``hi - lo`` of its window."""
    world, m, per = gathered.shape
    if n is None or n == world * per:
        if isinstance(gathered, np.ndarray):
            return np.ascontiguousarray(gathered.transpose(1, 0, 2)).reshape(m, world * per)
        return gathered.permute(1, 0, 2).reshape(m, world * per)
    parts = []
    for rank in range(world):
        lo, hi = shard_bounds(n, world, rank)
        parts.append(gathered[rank][:, :hi - lo])
    if isinstance(gathered, np.ndarray):
        return np.concatenate(parts, axis=1)
    import torch

    return torch.cat(parts, dim=1)


def widest_shard(n: int, world: int) -> int:
    """Columns of the widest shard: what the gather buffers are sized for."""
    return -(-n // world)


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


class _DeviceArray:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can view library-owned memory."""

    def __init__(self, ptr: int, shape: tuple, typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3}


class PeerGather:
    """Gathered results without a collective.

    Every rank owns one buffer that the other ranks map (CUDA inter-process handles exchanged over
    the process group, any backend): ``slots`` gathered results ``[world, m_max, n_shard]`` fp32 and
    one flag array per slot. :meth:`run` launches this rank's shard of a node: its kernels store
    the rank's columns into all ``world`` buffers and the last of their CTAs raises this rank's
    flag on every rank. With ``wait=True`` a one-warp kernel behind it waits for everybody's flag,
    and when the stream reaches the end of :meth:`run` the slot's local result is complete; with
    ``wait=False`` the caller puts :meth:`wait` where the results are first read, so consecutive
    nodes do not each pay a round trip between GPUs. Use at least two slots and alternate them,
    so that a fast rank writing step i+1 never touches what a slow rank still reads of step i.
    The layout arithmetic, the buffers and the calls live in the C++ helper
    (``kernels/parallel/peer_gather.h``); only the handle exchange uses the process group.
    """

    def __init__(self, dist, device_index: int, m_max: int, n_shard: int, slots: int = 2):
        import ctypes

        import torch

        from .._register import _host_lib, _raise_last

        self._ctypes, self._torch, self._raise = ctypes, torch, _raise_last
        self.lib = _host_lib()
        self.dist, self.device = dist, device_index
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        self.m_max, self.n_shard, self.slots = m_max, n_shard, slots
        handle = (ctypes.c_ubyte * 64)()
        self.own = self.lib.olc_peer_gather_create(self.world, self.rank, m_max, n_shard, slots, device_index, handle)
        if not self.own:
            _raise_last(1)
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle))
        table = (ctypes.c_ubyte * (64 * self.world)).from_buffer_copy(b"".join(handles))
        self._check(self.lib.olc_peer_gather_open(self.own, table))
        self._views = [torch.as_tensor(_DeviceArray(self.lib.olc_peer_gather_result(self.own, s),
                                                    (self.world, m_max, n_shard), "<f4"),
                                       device=torch.device("cuda", device_index)) for s in range(slots)]
        dist.barrier()

    def _check(self, code: int) -> None:
        if code != 0:
            self._raise(code)

    def result(self, slot: int):
        """Local gathered result of ``slot`` as a torch tensor ``[world, m_max, n_shard]`` (a view)."""
        return self._views[slot]

    def run(self, weights, a, slot: int, stream=None, accuracy_level: int = 0, wait: bool = True) -> None:
        """``weights``: this rank's :class:`MatMulNBitsWeights` shard; ``a`` [m, K] on this GPU.
        The step number is kept on the device, so the call can be captured in a CUDA graph."""
        torch = self._torch
        m = a.numel() // weights.k
        raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
        self._check(self.lib.olc_peer_gather_run(self.own, weights._handle, a.data_ptr(), m, accuracy_level, slot,
                                                 1 if wait else 0, raw))

    def wait(self, weights, slots, stream=None) -> None:
        """One small kernel: when the stream has passed it, the named slots hold every rank's
        columns of their last step. ``weights``: any node of this rank (its status word reports a
        wait that gave up)."""
        torch = self._torch
        slots = list(slots)
        raw = (stream or torch.cuda.current_stream(torch.device("cuda", self.device))).cuda_stream
        array = (self._ctypes.c_int * len(slots))(*slots)
        self._check(self.lib.olc_peer_gather_wait(self.own, weights._handle, array, len(slots), raw))

    def close(self) -> None:
        if self.own is None:
            return
        self._torch.cuda.synchronize()
        self.dist.barrier()   # nobody unmaps or frees while a peer may still store
        self.lib.olc_peer_gather_close_peers(self.own)
        self.dist.barrier()
        self.lib.olc_peer_gather_destroy(self.own)
        self.own = None
