"""The accuracy_level-4 entry point that never allocates (`mnb_matmul_int8_static`).

Some callers may not reach cudaMalloc while they run (a serving loop that must keep its steady
state free of allocation stalls and out-of-memory failures, a host that owns all device memory).
For them the quantized activations live in a fixed array inside the library instead of grown
scratch. The test calls the entry point through the C ABI twice in a row, with different
activations, and compares each result with the regular entry point. Collected last on purpose."""

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import _capi
from onnx_light_cpu_b200.tools import synthetic as syn

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
    for call, m in enumerate((16, 5)):  # the second call is smaller: stale bytes must not matter
        a_host = rng.standard_normal((m, case.k)).astype(np.float32) * (1.0 + call)
        a = torch.from_numpy(a_host).cuda()
        expect = torch.full((m, case.n), float("nan"), device="cuda")
        weights.matmul_device(a, expect, accuracy_level=4)
        got = torch.full((m, case.n), float("nan"), device="cuda")
        weights.matmul_int8_static(a, got)
        torch.cuda.synchronize()
        assert _capi.last_kernel().startswith("nbits_int8_matmul_kernel")
        assert rel_err(got.cpu().numpy(), expect.cpu().numpy()) <= TOL_FP32
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
