"""The accuracy_level-4 entry point that never allocates (`mnb_matmul_int8_static`).

Some callers may not reach cudaMalloc while they run (a serving loop that must keep its steady
state free of allocation stalls and out-of-memory failures, a host that owns all device memory).
For them the quantized activations live in a fixed array inside the library instead of grown
scratch. The test calls the entry point through the C ABI twice in a row, with different
activations, and compares each result with the regular entry point and with the CPU checker; the
free device memory must be the same before and after the steady-state calls. Collected last on
purpose."""

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import _capi
from onnx_light_cpu_b200.tools import synthetic as syn
from oracle import nbits_oracle as o

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5  # the tolerance of the other accuracy_level-4 output tests


def rel_err(y, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(y, dtype=np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def test_static_scratch_entry_matches_regular_entry_twice(cuda_device):
    import torch

    case = syn.make_case("static", 16, 4096, 300, 4, 32, seed=21, zero_points=True, bias=True)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n,
                                     bits=4, block_size=32)
    rng = np.random.default_rng(4)
    inputs = [rng.standard_normal((m, case.k)).astype(np.float32) * (1.0 + call)
              for call, m in enumerate((16, 5))]   # the second call is smaller: stale bytes must not matter
    on_device = [torch.from_numpy(a_host).cuda() for a_host in inputs]
    expects = [torch.full((a.shape[0], case.n), float("nan"), device="cuda") for a in on_device]
    gots = [torch.full((a.shape[0], case.n), float("nan"), device="cuda") for a in on_device]
    for a, expect in zip(on_device, expects):
        weights.matmul_device(a, expect, accuracy_level=4)
    # first call on this device: looks up the address of the built-in array (no allocation either)
    weights.matmul_int8_static(on_device[0], gots[0])
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info()
    for a, got in zip(on_device, gots):
        weights.matmul_int8_static(a, got)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, (free_before, free_after)   # the steady state took no device memory
    assert _capi.last_kernel().startswith("nbits_int8_matmul_kernel")
    for a_host, got, expect in zip(inputs, gots, expects):
        assert rel_err(got.cpu().numpy(), expect.cpu().numpy()) <= TOL_FP32
        reference = o.matmul_int8(a_host, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 32)
        assert rel_err(got.cpu().numpy(), reference) <= TOL_FP32
    weights.close()


def test_static_scratch_entry_rejects_host_memory(cuda_device):
    """A pointer the GPU cannot reach is an error code, not a device fault: the entry point checks
    where A and Y live like the other device-pointer entry points."""
    import ctypes

    import torch

    case = syn.make_case("static_host", 2, 256, 8, 4, 32, seed=24)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, None, K=256, N=8, bits=4, block_size=32)
    a_host = np.ascontiguousarray(case.a)
    y = torch.zeros((2, 8), device="cuda")
    status = _capi.load().mnb_matmul_int8_static(weights._handle, ctypes.c_void_p(a_host.ctypes.data), 2,
                                                 ctypes.c_void_p(y.data_ptr()), None)
    assert status == _capi.MNB_ERR_INVALID_ARGUMENT
    assert "mnb_matmul_host" in _capi.load().mnb_last_error().decode()
    weights.close()


def test_static_scratch_entry_rejects_sizes_beyond_its_array(cuda_device):
    import torch

    case = syn.make_case("static_big", 1, 32768, 8, 4, 128, seed=22)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, None, K=case.k, N=case.n,
                                     bits=4, block_size=128)
    a = torch.zeros((1, case.k), device="cuda")
    y = torch.zeros((1, case.n), device="cuda")
    with pytest.raises(_capi.MatMulNBitsError, match="exceed the built-in scratch") as info:
        weights.matmul_int8_static(a, y)
    assert info.value.status == _capi.MNB_ERR_INVALID_ARGUMENT
    small = syn.make_case("static_m", 17, 256, 8, 4, 32, seed=23)
    w2 = pkg.MatMulNBitsWeights(small.b, small.scales, small.zero_points, None, K=256, N=8, bits=4, block_size=32)
    with pytest.raises(_capi.MatMulNBitsError, match="exceed the built-in scratch"):
        w2.matmul_int8_static(torch.zeros((17, 256), device="cuda"), torch.zeros((17, 8), device="cuda"))
    weights.close()
    w2.close()
