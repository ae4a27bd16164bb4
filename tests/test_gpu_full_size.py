"""BASELINE configurations at their full sizes against the CPU checker on a random sample of
output columns (all rows of the sample): the checker is too slow for the full products, a
permutation of k or a mix-up of token tiles shows in any column.

Error measure used here, element by element (`assert_close`):

    |y - ref| <= tol * |ref| + tol * rms(ref row)

An output is a sum of K products of either sign, so an output near zero still carries the rounding
of K products whose size is that of the row's typical output: the second term is the floor a
cancelling sum has in ANY fp32 evaluation order (the fp32 checker itself sits at about 2e-7 of the
row's rms from the fp64 one). tol is the bar of the path: 1e-5 (decode), 2e-2 (bf16 tensor cores).
"""

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import _capi
from onnx_light_cpu_b200.tools import synthetic as syn
from oracle import nbits_oracle as o

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5
TOL_BF16 = 2e-2
SAMPLE = 64


def assert_close(y, ref, tol, what=""):
    y = np.asarray(y, dtype=np.float64)
    ref = np.asarray(ref, dtype=np.float64)
    rms = np.sqrt(np.mean(ref * ref, axis=-1, keepdims=True))
    excess = np.abs(y - ref) - (tol * np.abs(ref) + tol * rms)
    worst = np.unravel_index(np.argmax(excess), excess.shape)
    assert excess[worst] <= 0, (what, worst, float(y[worst]), float(ref[worst]), float(rms[worst[0], 0]))


def sampled_reference(case, columns, kind):
    """Checker output for the sampled columns only (their weight rows, scales, zero points, bias)."""
    nb = case.n_blocks
    b = np.ascontiguousarray(case.b[columns])
    scales = np.ascontiguousarray(case.scales.reshape(case.n, nb)[columns]).reshape(-1)
    zp = None if case.zero_points is None else np.ascontiguousarray(case.zero_points[columns])
    bias = None if case.bias is None else np.ascontiguousarray(case.bias[columns])
    fn = {"f64": o.matmul_f64, "bf16": o.matmul_bf16, "int8": o.matmul_int8}[kind]
    return fn(case.a, b, scales, zp, bias, len(columns), case.k, case.bits, case.block_size)


def run_full(case, accuracy_level=0, path=_capi.PATH_AUTO):
    import torch

    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n,
                                     bits=case.bits, block_size=case.block_size)
    a = torch.from_numpy(case.a).cuda()
    y = torch.full((case.m, case.n), float("nan"), device="cuda", dtype=torch.float32)
    weights.matmul_device(a, y, accuracy_level=accuracy_level, path=path)
    torch.cuda.synchronize()
    assert weights.poll_status() == 0
    kernel = _capi.last_kernel()
    out = y.cpu().numpy()
    weights.close()
    del a, y
    torch.cuda.empty_cache()
    return out, kernel


def sample_columns(case, seed):
    rng = np.random.default_rng(seed)
    columns = np.sort(rng.choice(case.n, size=min(SAMPLE, case.n), replace=False))
    columns[0], columns[-1] = 0, case.n - 1   # the edges of the first and the last tile
    return np.unique(columns)


# ---- cfg3: prefill on the bf16 tcgen05 path, every M of the configuration, full N -------------------
@pytest.mark.parametrize("m", [512, 2048, 8192])
def test_config3_prefill_full_size_sampled_columns(cuda_device, m):
    case = syn.config3(m)
    y, kernel = run_full(case)
    assert kernel.startswith("nbits_gemm_tcgen05"), kernel
    assert not np.isnan(y).any()
    columns = sample_columns(case, 300 + m)
    assert_close(y[:, columns], sampled_reference(case, columns, "bf16"), TOL_BF16, "bf16 model")
    assert_close(y[:, columns], sampled_reference(case, columns, "f64"), TOL_BF16, "exact")


# ---- cfg4: the seven projections of the layer at full N, both accuracy levels ----------------------
@pytest.mark.parametrize("accuracy_level", [0, 4])
@pytest.mark.parametrize("index", range(7))
def test_config4_layer_shapes_full_size_sampled_columns(cuda_device, index, accuracy_level):
    case = syn.config4(accuracy_level)[index]
    y, kernel = run_full(case, accuracy_level=accuracy_level)
    assert not np.isnan(y).any()
    columns = sample_columns(case, 400 + index)
    if accuracy_level == 4:
        assert kernel == "nbits_int8_mma_kernel", kernel
        assert_close(y[:, columns], sampled_reference(case, columns, "int8"), TOL_FP32, case.name)
    else:
        assert_close(y[:, columns], sampled_reference(case, columns, "f64"), TOL_FP32, case.name)


# ---- cfg5: one column shard of the large-N projection (N / 8 = 16032), 4 and 8 bit, M = 1, 8, 256 ---
@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("m", [1, 8, 256])
def test_config5_shard_full_size_sampled_columns(cuda_device, m, bits):
    case = syn.shard_columns(syn.config5(m, bits, n=128256 // 8 * 2), 2, 1)   # second of two shards: offsets matter
    assert case.n == 16032
    y, kernel = run_full(case)
    assert not np.isnan(y).any()
    columns = sample_columns(case, 500 + m + bits)
    if m > 16 and kernel.startswith("nbits_gemm_tcgen05"):
        assert_close(y[:, columns], sampled_reference(case, columns, "f64"), TOL_BF16, kernel)
    else:
        assert_close(y[:, columns], sampled_reference(case, columns, "f64"), TOL_FP32, kernel)


def test_config5_full_width_m1_sampled_columns(cuda_device):
    """The whole N = 128256 projection on one GPU (4-bit, M = 1): 337 MB of operands."""
    case = syn.config5(1, 4)
    y, kernel = run_full(case)
    assert not np.isnan(y).any()
    columns = sample_columns(case, 77)
    assert_close(y[:, columns], sampled_reference(case, columns, "f64"), TOL_FP32, kernel)


# ---- cfg2 and cfg1 at full size, element by element (every column) ---------------------------------
@pytest.mark.parametrize("m", [1, 4, 16])
def test_config2_element_wise(cuda_device, m):
    case = syn.config2(m)
    y, kernel = run_full(case)
    assert_close(y, o.matmul_f64(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 128),
                 TOL_FP32, kernel)


def test_config1_element_wise(cuda_device):
    case = syn.config1()
    y, kernel = run_full(case)
    assert_close(y, o.matmul_f64(case.a, case.b, case.scales, None, None, case.n, case.k, 4, 32), TOL_FP32, kernel)
