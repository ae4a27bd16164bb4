"""Column-sharded decode whose kernel stores its columns into every rank's gathered result through
peer-mapped memory (no collective). Needs two GPUs on one box; runs as two child processes, one per
GPU, that exchange the buffer handles over a gloo process group."""

import os
import socket

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5
TOL_BF16 = 2e-2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int) -> None:
    import torch
    import torch.distributed as dist

    import onnx_light_cpu_b200 as pkg
    from onnx_light_cpu_b200.tools import sharded
    from onnx_light_cpu_b200.tools import synthetic as syn
    from oracle import nbits_oracle as o

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # (bits, block, N, tokens per step, accuracy_level, wait inside run): the decode kernels store to
        # the peers themselves; 8-bit weights, more tokens and accuracy_level 4 go through the ordinary
        # dispatch and the kernel that copies the local window to the peers. N = 645 does not divide
        # by two ranks: shards of 323 and 322 columns in windows of 323.
        for bits, bs, n, ms, level, wait in ((4, 128, 2048, (1, 3, 8, 1), 0, True), (4, 32, 640, (1, 2, 1), 0, True),
                                             (4, 32, 640, (1, 8, 2), 0, False), (8, 32, 640, (1, 8), 0, False),
                                             (4, 64, 1024, (40, 24), 0, True), (4, 32, 1024, (16, 5), 4, False),
                                             (4, 128, 645, (1, 4, 1), 0, False)):
            k = 4096
            case = syn.make_case("peer", max(ms), k, n, bits, bs, seed=77 + bs + bits, zero_points=True, bias=True)
            lo, hi = sharded.shard_bounds(n, world, rank)
            width = sharded.widest_shard(n, world)
            nb = k // bs
            weights = pkg.MatMulNBitsWeights(case.b[lo:hi], case.scales.reshape(n, nb)[lo:hi].reshape(-1),
                                             case.zero_points[lo:hi], case.bias[lo:hi], K=k, N=hi - lo, bits=bits,
                                             block_size=bs, device=rank)
            gather = sharded.PeerGather(dist, rank, m_max=max(ms), n_shard=width, slots=2)
            for step, m in enumerate(ms):
                a_host = (case.a[:m] * (1.0 + step)).astype(np.float32)
                a = torch.from_numpy(a_host).cuda()
                slot = step % 2
                gather.run(weights, a, slot, accuracy_level=level, wait=wait)
                if not wait:
                    gather.wait(weights, [slot])
                torch.cuda.synchronize()
                assert weights.poll_status() == 0
                got = sharded.assemble(gather.result(slot)[:, :m, :], n=n).cpu().numpy()
                if level == 4:
                    ref = o.matmul_int8(a_host, case.b, case.scales, case.zero_points, case.bias, n, k, bits, bs)
                else:
                    ref = o.matmul_f64(a_host, case.b, case.scales, case.zero_points, case.bias, n, k, bits, bs)
                err = float(np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30))
                tol = TOL_BF16 if (m > 16 and level == 0) else TOL_FP32
                assert err <= tol, (rank, bits, bs, step, m, level, err)
                dist.barrier()   # the host check of this step is over on every rank
            gather.close()
            weights.close()
    finally:
        dist.destroy_process_group()


def test_gather_entry_point_single_rank():
    """World size 1: the entry point, the flag exchange and the buffer views without any peer."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(1, _free_port()), nprocs=1, join=True)


def test_peer_store_gather_two_gpus():
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(2, _free_port()), nprocs=2, join=True)


def test_device_entry_point_refuses_memory_of_another_gpu():
    """Weights on GPU 0, activations on GPU 1: an error code, not a fault."""
    import torch

    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs on one box")
    import onnx_light_cpu_b200 as pkg
    from onnx_light_cpu_b200 import _capi
    from onnx_light_cpu_b200.tools import synthetic as syn

    case = syn.make_case("wrong_gpu", 1, 4096, 64, 4, 128, seed=3)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=4096, N=64, bits=4, block_size=128, device=0)
    a = torch.from_numpy(case.a).to("cuda:1")
    y = torch.zeros((1, 64), device="cuda:1")
    # the Python wrapper refuses the tensors, and the C entry point refuses the raw addresses
    with pytest.raises(ValueError, match="the weights are on GPU 0"):
        weights.matmul_device(a, y)
    with pytest.raises(_capi.MatMulNBitsError, match="must be memory of GPU 0") as info:
        _capi.check(weights._lib.mnb_matmul_device_strided(
            weights._handle, a.data_ptr(), 1, 0, _capi.PATH_AUTO, y.data_ptr(), 64, 0,
            torch.cuda.current_stream(0).cuda_stream))
    assert info.value.status == _capi.MNB_ERR_INVALID_ARGUMENT
    weights.close()


def test_gather_wait_gives_up_and_reports(cuda_device):
    """Failure detection without a fault: a gathered step whose second "rank" never raises its flag
    (both ranks' buffers are plain local memory here, nobody plays rank 1). The bounded wait of the
    flag exchange runs out after about a second, the kernel returns, the status word reads 5
    (peer flag) once and 0 afterwards, and the context is usable: an ordinary product is correct."""
    import ctypes

    import torch

    import onnx_light_cpu_b200 as pkg
    from onnx_light_cpu_b200 import _capi
    from onnx_light_cpu_b200.tools import synthetic as syn
    from oracle import nbits_oracle as o

    case = syn.make_case("gather_timeout", 1, 4096, 256, 4, 128, seed=31, bias=True)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n, bits=4,
                                     block_size=128)
    a = torch.from_numpy(case.a).cuda()
    results = [torch.zeros((1, case.n), device="cuda") for _ in range(2)]
    flags = [torch.zeros(_capi.MAX_GATHER_RANKS + 1, dtype=torch.int32, device="cuda") for _ in range(2)]
    y_ranks = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in results])
    flag_ranks = (ctypes.c_void_p * 2)(*[t.data_ptr() for t in flags])
    raw = torch.cuda.current_stream().cuda_stream
    _capi.check(_capi.load().mnb_matmul_device_gather(weights._handle, a.data_ptr(), 1, y_ranks, flag_ranks, 2, 0,
                                                      case.n, 0, 1, raw))
    assert weights.poll_status() == 5       # kDeviceTimeoutPeerFlag; the poll waits for the device
    assert weights.poll_status() == 0       # read once, then cleared
    ref = o.matmul_f64(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 128)
    for got in results:                     # the columns were stored into both buffers before the wait
        err = float(np.abs(got.cpu().numpy() - ref).max() / np.abs(ref).max())
        assert err <= TOL_FP32
    assert int(flags[1][0].item()) == 1     # this rank's flag was raised on the "peer"
    y = torch.zeros((1, case.n), device="cuda")
    weights.matmul_device(a, y)
    torch.cuda.synchronize()
    assert weights.poll_status() == 0
    assert float(np.abs(y.cpu().numpy() - ref).max() / np.abs(ref).max()) <= TOL_FP32
    weights.close()
