"""Sibling nodes that take the same activations through one call (`mnb_matmul_device_group`), and
the seven-node decoder-layer driver built on it, against the CPU checker."""

import ctypes

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import _capi
from onnx_light_cpu_b200.matmul_nbits import matmul_device_group
from onnx_light_cpu_b200.tools import synthetic as syn
from oracle import nbits_oracle as o

from test_gpu_full_size import assert_close, sample_columns, sampled_reference

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5


def make_nodes(shapes, k, block_size, *, zero_points, bias, m, seed, a_seed=None):
    """Cases of sibling nodes: own weights each, the activations of the first one for all."""
    cases = [syn.make_case(f"group{i}", m, k, n, 4, block_size, seed=seed + i,
                           zero_points=zero_points if isinstance(zero_points, bool) else zero_points[i],
                           bias=bias, scale_sigma=0.01, fp16_a=True)
             for i, n in enumerate(shapes)]
    for case in cases[1:]:
        case.a = cases[0].a
    return cases


def upload(cases):
    return [pkg.MatMulNBitsWeights(c.b, c.scales, c.zero_points, c.bias, K=c.k, N=c.n, bits=c.bits,
                                   block_size=c.block_size) for c in cases]


def run_group(cases, accuracy_level=0, single_path=_capi.PATH_AUTO):
    import torch

    nodes = upload(cases)
    a = torch.from_numpy(cases[0].a).cuda()
    ys = [torch.full((c.m, c.n), float("nan"), device="cuda") for c in cases]
    torch.cuda.synchronize()
    before = _capi.launch_count()
    matmul_device_group(nodes, a, ys, accuracy_level=accuracy_level)
    torch.cuda.synchronize()
    launches = _capi.launch_count() - before
    kernel = _capi.last_kernel()
    assert all(node.poll_status() == 0 for node in nodes)
    singles = [torch.full((c.m, c.n), float("nan"), device="cuda") for c in cases]
    for node, y in zip(nodes, singles):
        node.matmul_device(a, y, accuracy_level=accuracy_level, path=single_path)
    torch.cuda.synchronize()
    out = [y.cpu().numpy() for y in ys]
    alone = [y.cpu().numpy() for y in singles]
    for node in nodes:
        node.close()
    return out, alone, kernel, launches


@pytest.mark.parametrize("shapes,k,zp,bias", [
    ((2048, 1032), 4096, True, True),        # two nodes, the second ends in a short tile group and a short tile
    ((4096, 1024, 1024), 4096, False, False),  # q / k / v
    ((264, 8, 520), 2048, True, False),      # a node of a single tile in the middle
    ((14336, 14336), 4096, True, True),      # gate / up at full size: several rounds per CTA
])
def test_one_token_group_is_one_resident_launch(cuda_device, shapes, k, zp, bias):
    cases = make_nodes(shapes, k, 128, zero_points=zp, bias=bias, m=1, seed=9100 + len(shapes) + k)
    # (alone: the same kernel on request; AUTO would send the narrow nodes to the direct kernel)
    out, alone, kernel, launches = run_group(cases, single_path=_capi.PATH_GEMV_RESIDENT)
    assert kernel == "nbits_decode_resident_kernel", kernel
    assert launches == 1
    for case, y, y1 in zip(cases, out, alone):
        assert not np.isnan(y).any()
        if case.n > 4096:
            columns = sample_columns(case, 77)
            assert_close(y[:, columns], sampled_reference(case, columns, "f64"), TOL_FP32, case.name)
        else:
            ref = o.matmul_f64(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 128)
            assert_close(y, ref, TOL_FP32, case.name)
        # the same arithmetic per tile as the single-node launch
        np.testing.assert_array_equal(y, y1)


def test_one_token_group_of_mixed_nodes_runs_node_by_node(cuda_device):
    """Zero points in one node only: no shared kernel, same results as separate calls."""
    cases = make_nodes((512, 520), 4096, 128, zero_points=(True, False), bias=True, m=1, seed=9200)
    out, alone, _, launches = run_group(cases)
    assert launches == 2
    for case, y, y1 in zip(cases, out, alone):
        ref = o.matmul_f64(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 128)
        assert_close(y, ref, TOL_FP32, case.name)
        np.testing.assert_array_equal(y, y1)


@pytest.mark.parametrize("m", [5, 16])
@pytest.mark.parametrize("accuracy_level", [0, 4])
def test_small_block_group_shares_its_prologue(cuda_device, m, accuracy_level):
    """Block size 32, several tokens: what the nodes share is done once and their row tiles form one
    sequence over the CTAs of a single product launch."""
    cases = make_nodes((1024, 272, 528), 2048, 32, zero_points=False, bias=True, m=m, seed=9300 + m)
    import torch

    nodes = upload(cases)
    a = torch.from_numpy(cases[0].a).cuda()
    ys = [torch.full((c.m, c.n), float("nan"), device="cuda") for c in cases]
    before = _capi.launch_count()
    matmul_device_group(nodes, a, ys, accuracy_level=accuracy_level)
    torch.cuda.synchronize()
    launches = _capi.launch_count() - before
    # level 4: the quantization and ONE product launch for the three nodes; level 0: the digit rows, ONE
    # product launch, then the sum of the slices per node
    expected = 2 if accuracy_level == 4 else 5
    assert launches == expected, launches
    for case, node, y in zip(cases, nodes, ys):
        assert node.poll_status() == 0
        got = y.cpu().numpy()
        fn = o.matmul_int8 if accuracy_level == 4 else o.matmul_f64
        ref = fn(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 32)
        assert_close(got, ref, TOL_FP32, case.name)
        alone = torch.full((case.m, case.n), float("nan"), device="cuda")
        node.matmul_device(a, alone, accuracy_level=accuracy_level)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got, alone.cpu().numpy())
        node.close()


@pytest.mark.parametrize("accuracy_level", [0, 4])
@pytest.mark.parametrize("shapes,k,bs,zp", [
    ((77, 8, 100), 2048, 32, True),        # ragged N in every node: row tiles end at node boundaries
    ((4096, 1024, 1024), 4096, 32, False),  # q / k / v of the layer at full size
    ((520, 264), 14336, 128, True),         # seven K slices
])
def test_grouped_product_launch_matches_separate_calls(cuda_device, shapes, k, bs, zp, accuracy_level):
    """Sixteen tokens: one product launch over the nodes' row tiles gives, bit for bit, what one call per
    node gives, and both match the checker."""
    cases = make_nodes(shapes, k, bs, zero_points=zp, bias=True, m=16, seed=9500 + k + bs)
    out, alone, kernel, launches = run_group(cases, accuracy_level=accuracy_level)
    assert kernel == ("nbits_int8_mma_kernel" if accuracy_level == 4 else "nbits_digits_mma_kernel"), kernel
    assert launches == (2 if accuracy_level == 4 else 2 + len(shapes))
    kind = "int8" if accuracy_level == 4 else "f64"
    for case, y, y1 in zip(cases, out, alone):
        assert not np.isnan(y).any()
        np.testing.assert_array_equal(y, y1)
        columns = sample_columns(case, 91)
        assert_close(y[:, columns], sampled_reference(case, columns, kind), TOL_FP32, case.name)


def test_group_entry_refuses_bad_groups(cuda_device):
    import torch

    cases = make_nodes((64, 64), 1024, 128, zero_points=False, bias=False, m=1, seed=9400)
    other_k = syn.make_case("other_k", 1, 2048, 64, 4, 128, seed=9401, zero_points=False)
    nodes = upload(cases + [other_k])
    a = torch.from_numpy(cases[0].a).cuda()
    ys = [torch.zeros((1, 64), device="cuda") for _ in range(4)]
    lib = nodes[0]._lib

    def call(handles, outputs, m=1, level=0):
        hs = (ctypes.c_void_p * max(1, len(handles)))(*handles)
        os_ = (ctypes.c_void_p * max(1, len(outputs)))(*[y.data_ptr() for y in outputs])
        return lib.mnb_matmul_device_group(hs, len(handles), a.data_ptr(), m, level, os_, None)

    h = [node._handle for node in nodes]
    assert call([], []) == _capi.MNB_ERR_INVALID_ARGUMENT
    assert call([h[0]] * 4, ys) == _capi.MNB_ERR_INVALID_ARGUMENT
    assert call([h[0], h[0]], ys[:2]) == _capi.MNB_ERR_INVALID_ARGUMENT          # a node twice
    assert call([h[0], h[1]], [ys[0], ys[0]]) == _capi.MNB_ERR_INVALID_ARGUMENT  # an output twice
    assert call([h[0], h[2]], ys[:2]) == _capi.MNB_ERR_INVALID_ARGUMENT          # different K
    assert call([h[0], h[1]], ys[:2], level=3) == _capi.MNB_ERR_INVALID_ARGUMENT
    assert call([h[0], h[1]], ys[:2], m=-1) == _capi.MNB_ERR_INVALID_ARGUMENT
    assert call([h[0], h[1]], ys[:2], m=0) == _capi.MNB_OK
    with pytest.raises(ValueError):
        matmul_device_group(nodes[:2], a, ys[:1])
    with pytest.raises(ValueError):
        matmul_device_group([nodes[0], nodes[2]], a, ys[:2])
    assert call([h[0], h[1]], ys[:2]) == _capi.MNB_OK
    torch.cuda.synchronize()
    for node in nodes:
        node.close()


@pytest.mark.parametrize("accuracy_level", [0, 4])
def test_decoder_layer_driver_full_size_sampled_columns(cuda_device, accuracy_level):
    """All seven projections of benchmark configuration 4 (M = 16) through the layer driver."""
    import torch

    from onnx_light_cpu_b200.tools.decoder_layer import STAGES, DecoderLayerProjections

    layer = DecoderLayerProjections.synthetic(16, accuracy_level)
    inputs = layer.inputs_from_cases()
    outs = layer.run(inputs, accuracy_level=accuracy_level)
    torch.cuda.synchronize()
    assert layer.poll_status() == 0
    kind = "int8" if accuracy_level == 4 else "f64"
    for key, names in STAGES:
        for name in names:
            case = layer.cases[name]
            case.a = layer.cases[names[0]].a   # the stage's activations
            y = outs[name].cpu().numpy()
            assert not np.isnan(y).any()
            columns = sample_columns(case, 600 + len(name))
            assert_close(y[:, columns], sampled_reference(case, columns, kind), TOL_FP32, name)
    assert layer.algorithmic_bytes(16) > 136_000_000
    layer.close()
