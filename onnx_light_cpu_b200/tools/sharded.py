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


class _DeviceArray:
    """Minimal ``__cuda_array_interface__`` carrier so that torch can view library-owned memory."""

    def __init__(self, ptr: int, shape: tuple, typestr: str):
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3}


class PeerGather:
    """Gathered decode results without a collective.

    Every rank owns one buffer that the other ranks map (CUDA inter-process handles exchanged over
    the process group, any backend): ``slots`` gathered results ``[world, m_max, n_shard]`` fp32 and
    one flag array per slot. :meth:`run` launches the decode kernel, which stores this rank's
    columns into all ``world`` buffers, and a one-warp kernel that raises this rank's flag on every
    rank and waits for everybody's flag locally. When the stream reaches the end of :meth:`run`
    the slot's local result is complete. Use at least two slots and alternate them, so that a fast
    rank writing step i+1 never touches what a slow rank still reads of step i.
    """

    def __init__(self, dist, device_index: int, m_max: int, n_shard: int, slots: int = 2):
        import ctypes

        import torch

        from onnx_light_cpu_b200 import _capi

        self._capi, self._ctypes, self._torch = _capi, ctypes, torch
        self.lib = _capi.load()
        self.dist, self.device = dist, device_index
        self.world, self.rank = dist.get_world_size(), dist.get_rank()
        if self.world > _capi.MAX_GATHER_RANKS:
            raise ValueError(f"at most {_capi.MAX_GATHER_RANKS} ranks")
        self.m_max, self.n_shard, self.slots = m_max, n_shard, slots
        self.slot_floats = self.world * m_max * n_shard
        self.flags_offset = (slots * self.slot_floats * 4 + 255) // 256 * 256
        self.bytes = self.flags_offset + slots * 256
        own = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * _capi.IPC_HANDLE_BYTES)()
        _capi.check(self.lib.mnb_peer_buffer_create(device_index, self.bytes, ctypes.byref(own), handle))
        self.own = own.value
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle))
        self.bases = []
        for r, raw in enumerate(handles):
            if r == self.rank:
                self.bases.append(self.own)
                continue
            ptr = ctypes.c_void_p()
            buf = (ctypes.c_ubyte * _capi.IPC_HANDLE_BYTES).from_buffer_copy(raw)
            _capi.check(self.lib.mnb_peer_buffer_open(device_index, buf, ctypes.byref(ptr)))
            self.bases.append(ptr.value)
        self._views = [torch.as_tensor(_DeviceArray(self.own + s * self.slot_floats * 4,
                                                    (self.world, m_max, n_shard), "<f4"),
                                       device=torch.device("cuda", device_index)) for s in range(slots)]
        dist.barrier()

    def result(self, slot: int):
        """Local gathered result of ``slot`` as a torch tensor ``[world, m_max, n_shard]`` (a view)."""
        return self._views[slot]

    def run(self, weights, a, slot: int, stream=None) -> None:
        """``weights``: this rank's :class:`MatMulNBitsWeights` shard; ``a`` [m, K] on this GPU.
        The step number is kept on the device, so the call can be captured in a CUDA graph."""
        c, torch = self._ctypes, self._torch
        m = a.numel() // weights.k
        if m > self.m_max or weights.n != self.n_shard:
            raise ValueError("shape does not match the gather buffers")
        window = (slot * self.world + self.rank) * self.m_max * self.n_shard * 4
        y_ranks = (c.c_void_p * self.world)(*[base + window for base in self.bases])
        flags = (c.c_void_p * self.world)(*[base + self.flags_offset + slot * 256 for base in self.bases])
        raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
        self._capi.check(self.lib.mnb_matmul_device_gather(
            weights._handle, a.data_ptr(), m, y_ranks, flags, self.world, self.rank, self.n_shard, 0, 0, raw))

    def close(self) -> None:
        if self.own is None:
            return
        self._torch.cuda.synchronize()
        self.dist.barrier()   # nobody unmaps or frees while a peer may still store
        for r, base in enumerate(self.bases):
            if r != self.rank:
                self.lib.mnb_peer_buffer_close(self.device, base)
        self.dist.barrier()
        self.lib.mnb_peer_buffer_destroy(self.device, self.own)
        self.own = None
