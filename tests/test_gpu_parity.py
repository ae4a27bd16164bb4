"""Parity of the CUDA path with the CPU checker, through the C ABI (device pointers) and
through the registered operator (host tensors). Bars:
  * integer dequantization and int32 block dots: bit-exact
  * CUDA-core fp32 decode path: max |y - y_ref| / max |y_ref| <= 1e-5
  * bf16 tensor-core path:      max |y - y_ref| / max |y_ref| <= 2e-2
"""

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import _capi
from onnx_light_cpu_b200.matmul_nbits import quantize_a
from onnx_light_cpu_b200.tools import synthetic as syn
from oracle import nbits_oracle as o

pytestmark = pytest.mark.gpu

TOL_FP32 = 1e-5
TOL_BF16 = 2e-2


def rel_err(y, ref):
    ref = np.asarray(ref, dtype=np.float64)
    return float(np.abs(np.asarray(y, dtype=np.float64) - ref).max() / max(np.abs(ref).max(), 1e-30))


def run_device(case, path=_capi.PATH_AUTO, accuracy_level=0):
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
    return out, kernel


DIRECT = "nbits_decode_direct_kernel"
RESIDENT = "nbits_decode_resident_kernel"


def resident_takes(case):
    """Shapes AUTO sends to the one-token kernel that asks for all of its weights at kernel start."""
    blocks = -(-case.k // case.block_size)
    # long rows, or few tiles per CTA with rows that are not short, leave the tile-per-warp kernel too few warps
    if case.k > 4096 or not (case.n >= 4736 or (case.k <= 2048 and (case.block_size == 32 or case.n >= 4096))):
        return False
    if case.bits == 4 and case.block_size == 32 and case.m == 1:
        return case.k % 1024 == 0      # blocks of 32: whole chunks of 32 scales per row
    return (case.bits == 4 and case.block_size == 128 and case.m == 1 and blocks % 8 == 0 and
            (case.zero_points is None or blocks % 16 == 0))


def direct_takes(case):
    """Shapes AUTO sends to the direct-stream decode kernel: one token, 4-bit, block 128, blocks per
    row a multiple of four (and the resident kernel does not take them)."""
    return (case.bits == 4 and case.block_size == 128 and case.m == 1 and
            (-(-case.k // case.block_size)) % 4 == 0 and not resident_takes(case))


def sliced_digits_take(case):
    """Shapes AUTO sends to the one-pass digit kernel: five to sixteen tokens (three and four too on
    rows of 8192 k and more), 4-bit, packed rows that are whole 128-byte units."""
    m, bs = case.m, case.block_size
    enough_tokens = 5 <= m <= 16 or (3 <= m <= 16 and case.k >= 8192)   # long rows: from three tokens on
    return case.bits == 4 and enough_tokens and (case.k // 2) % 128 == 0 and 32 <= bs <= 1024


SLICED = "nbits_digits_mma_kernel"


def oracle_f64(case):
    return o.matmul_f64(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, case.bits,
                        case.block_size)


# ---- integer dequantization: bit-exact ---------------------------------------------------------
@pytest.mark.parametrize("bits,bs,k,n,zp", [(4, 32, 4096, 64, False), (4, 128, 4096, 96, True), (4, 16, 80, 7, True),
                                            (4, 64, 200, 5, True), (8, 32, 4096, 33, True), (8, 16, 40, 3, False)])
def test_dequant_integers_bit_exact(cuda_device, bits, bs, k, n, zp):
    import torch

    case = syn.make_case("dq", 1, k, n, bits, bs, seed=11 + bits + bs, zero_points=zp)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, None, K=k, N=n, bits=bits, block_size=bs)
    out = torch.empty((n, k), dtype=torch.int32, device="cuda")
    weights.dequant_int(out)
    torch.cuda.synchronize()
    assert np.array_equal(out.cpu().numpy(), o.dequant_int(case.b, case.zero_points, n, k, bits, bs))


# ---- decode path -----------------------------------------------------------------------------------
def test_config1_single_node(cuda_device):
    case = syn.config1()
    y, kernel = run_device(case)
    assert kernel == "nbits_gemv_mma_kernel", kernel   # fewer than four tiles per CTA: the fp16 two-piece kernel
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32
    assert rel_err(y, o.matmul_f32(case.a, case.b, case.scales, None, None, case.n, case.k, 4, 32)) <= TOL_FP32
    y1, kernel1 = run_device(case, path=_capi.PATH_GEMV_RESIDENT)
    assert kernel1 == RESIDENT, kernel1    # on request: one integer MMA per block of 32
    assert rel_err(y1, oracle_f64(case)) <= TOL_FP32
    y2, kernel2 = run_device(case, path=_capi.PATH_GEMV)
    assert kernel2.startswith("nbits_gemv_stream_kernel<4,1,"), kernel2
    assert rel_err(y2, oracle_f64(case)) <= TOL_FP32


@pytest.mark.parametrize("m", [1, 4, 16])
def test_config2_decode_sweep(cuda_device, m):
    case = syn.config2(m)
    y, kernel = run_device(case)
    expected = {1: RESIDENT, 4: "nbits_gemv_mma_kernel", 16: SLICED}[m]
    assert kernel == expected, kernel
    ref = oracle_f64(case)
    assert rel_err(y, ref) <= TOL_FP32
    y2, kernel2 = run_device(case, path=_capi.PATH_GEMV)
    assert kernel2.startswith("nbits_gemv_stream_kernel"), kernel2
    assert rel_err(y2, ref) <= TOL_FP32


DECODE_EDGES = [
    # m, k, n, bits, block, zp, bias
    (1, 4096, 1, 4, 32, True, True),        # single column
    (3, 4096, 149, 4, 64, True, False),     # N not a multiple of any tile, odd M
    (2, 1024, 300, 4, 32, False, True),     # narrow rows: 16 row groups
    (1, 14336, 64, 4, 32, True, False),     # wide K: one row group, idle lanes
    (5, 8192, 40, 4, 256, True, True),
    (1, 20480, 24, 4, 128, True, False),    # two chunk columns per thread
    (1, 4096, 77, 8, 32, True, True),       # 8-bit
    (7, 4096, 50, 8, 128, False, False),
    (16, 2048, 31, 8, 16, True, True),
    (1, 4000, 33, 4, 32, True, True),       # K not a multiple of the chunk: word-wise kernel
    (2, 96, 5, 4, 16, True, False),         # block 16: word-wise kernel
    (1, 40, 3, 8, 32, True, True),          # partial last block
    (16, 4096, 2, 4, 128, True, True),
]


@pytest.mark.parametrize("path", [_capi.PATH_AUTO, _capi.PATH_GEMV])
@pytest.mark.parametrize("m,k,n,bits,bs,zp,bias", DECODE_EDGES)
def test_decode_edge_cases(cuda_device, m, k, n, bits, bs, zp, bias, path):
    case = syn.make_case("edge", m, k, n, bits, bs, seed=m * 7 + k + n + bits, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=path)
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32, kernel


MMA_CASES = [
    # m, k, n, block, zp, bias
    (1, 4096, 4096, 32, False, False),     # cfg1 geometry
    (1, 4096, 1024, 128, True, True),      # cfg2 geometry, reduced N
    (4, 4096, 1000, 128, True, True),      # four tokens in one pass, N not a multiple of 8
    (16, 4096, 200, 128, True, False),     # four passes
    (2, 4096, 333, 64, True, True),        # two blocks per supergroup
    (3, 2048, 77, 64, False, True),        # two passes of two tokens
    (1, 14336, 96, 32, True, False),       # wide K, small blocks
    (2, 4096, 40, 32, True, True),         # one token per pass
    (1, 4096, 130, 256, True, True),       # block spans two supergroups
    (4, 8192, 64, 1024, False, False),
    (1, 4000, 50, 32, True, True),         # K not a multiple of 128: partial last supergroup
    (1, 4096 + 64, 24, 128, True, False),  # partial last block
    (1, 4096, 7, 128, True, True),         # fewer rows than one half tile
    (1, 4096, 14336, 128, True, True),     # cfg2 at full size: many tiles per CTA, slot ring wraps
    (2, 4096, 16032, 32, True, False),     # one lm-head shard: long ring, two passes
]

# shapes with more tokens than one column tile holds: (m, k, n, block, zp, bias)
MMA_MULTI_CASES = [
    (2, 4096, 16032, 32, True, False),     # one lm-head shard: long ring, two column tiles
    (8, 4096, 200, 128, True, True),       # two column tiles of four tokens, one pass
    (16, 2048, 100, 128, False, True),     # four column tiles, one pass
    (13, 4096, 120, 128, True, False),     # two passes of two column tiles, last one ragged
    (4, 4096, 64, 32, False, True),        # four column tiles of one token
    (16, 4096, 40, 32, True, True),        # four passes of four tokens
    (5, 4096, 77, 64, True, True),         # three of four column tiles of two tokens in use
    (8, 4096, 48, 512, False, False),      # block spans four supergroups, two column tiles
    (7, 4096, 14336, 128, True, True),     # full size with seven tokens
]


@pytest.mark.parametrize("m,k,n,bs,zp,bias", MMA_CASES)
def test_decode_mma_path(cuda_device, m, k, n, bs, zp, bias):
    case = syn.make_case("mma", m, k, n, 4, bs, seed=m * 11 + k + n + bs, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_MMA)
    assert kernel == "nbits_gemv_mma_kernel"
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32


@pytest.mark.parametrize("m,k,n,bs,zp,bias", MMA_MULTI_CASES)
def test_decode_mma_multi_tile_path(cuda_device, m, k, n, bs, zp, bias):
    case = syn.make_case("mma_multi", m, k, n, 4, bs, seed=m * 11 + k + n + bs, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_MMA_MULTI)
    assert kernel == "nbits_gemv_mma_multi_kernel"
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32
    y_auto, kernel_auto = run_device(case)
    if direct_takes(case):
        assert kernel_auto == DIRECT and rel_err(y, y_auto) <= TOL_FP32
    elif sliced_digits_take(case):
        # AUTO sends many tokens through the one-pass digit kernel
        assert kernel_auto == SLICED and rel_err(y, y_auto) <= TOL_FP32
    else:   # AUTO picks the same kernel for these shapes
        assert kernel_auto == kernel and np.array_equal(y, y_auto)
    y_single, _ = run_device(case, path=_capi.PATH_GEMV_MMA)   # one column tile per pass
    assert rel_err(y, y_single) <= TOL_FP32


def test_decode_mma_multi_tile_path_rejects_single_tile_shapes(cuda_device):
    import torch

    case = syn.make_case("mma_multi_reject", 3, 4096, 64, 4, 128, seed=8)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=4096, N=64, bits=4, block_size=128)
    with pytest.raises(_capi.MatMulNBitsError) as info:
        weights.matmul_device(torch.from_numpy(case.a).cuda(), torch.zeros((3, 64), device="cuda"),
                              path=_capi.PATH_GEMV_MMA_MULTI)
    assert info.value.status == _capi.MNB_ERR_UNSUPPORTED
    weights.close()


def test_decode_mma_path_wide_dynamic_range(cuda_device):
    """Activations spanning many orders of magnitude, large and tiny rows: the per-row power-of-two
    scaling keeps the two-piece fp16 split accurate."""
    case = syn.make_case("mma_range", 4, 4096, 256, 4, 128, seed=99, bias=True)
    rng = np.random.default_rng(1)
    case.a[0] *= 1e4
    case.a[1] *= 1e-6
    case.a[2] *= np.exp(rng.uniform(-8, 8, size=case.k)).astype(np.float32)
    case.a[3] = 0.0
    y, _ = run_device(case, path=_capi.PATH_GEMV_MMA)
    ref = oracle_f64(case)
    for row in range(3):
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    assert np.array_equal(y[3], case.bias)


# shapes for the integer-digit decode kernel: (m, k, n, block, zp, bias)
IMMA_CASES = [
    (1, 4096, 96, 128, True, True),        # whole-row tasks, two slices
    (2, 4096, 200, 128, False, True),      # two tokens = six MMA columns; signed codes (no zero points)
    (1, 2048, 77, 128, True, False),       # whole-row tasks, one slice: the odd warp of a pair idles
    (3, 4096, 130, 256, True, True),       # two passes, block spans two supergroups
    (1, 8192, 64, 1024, False, False),     # sliced tasks through the 2-D box, block spans eight supergroups
    (2, 14336, 48, 128, True, True),       # wide K: seven slices
    (1, 4096 + 64, 24, 128, True, False),  # partial last block, rows not whole tasks
    (1, 4000, 50, 128, True, True),        # K not a multiple of 128
    (1, 4096, 7, 128, True, True),         # fewer rows than one half tile
    (5, 4096, 40, 512, True, False),       # three passes, last one with a single token
    (1, 4096, 14336, 128, True, True),     # cfg2 at full size: seven tiles in six slots for some CTAs
    (2, 4096, 14336, 128, False, True),
]


@pytest.mark.parametrize("m,k,n,bs,zp,bias", IMMA_CASES)
def test_decode_imma_path(cuda_device, m, k, n, bs, zp, bias):
    case = syn.make_case("imma", m, k, n, 4, bs, seed=m * 13 + k + n + bs, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_IMMA)
    assert kernel == "nbits_gemv_imma_kernel"
    ref = oracle_f64(case)
    for row in range(m):   # every token against its own magnitude
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    y_mma, _ = run_device(case, path=_capi.PATH_GEMV_MMA)   # the fp16 two-piece kernel agrees
    assert rel_err(y, y_mma) <= TOL_FP32
    if m <= 2:
        y_auto, kernel_auto = run_device(case)   # AUTO: the resident / direct-stream kernels where they fit, else this one
        if resident_takes(case):
            assert kernel_auto == RESIDENT and rel_err(y, y_auto) <= TOL_FP32
        elif direct_takes(case):
            assert kernel_auto == DIRECT and rel_err(y, y_auto) <= TOL_FP32
        else:
            assert kernel_auto == kernel and np.array_equal(y, y_auto)


def test_decode_imma_path_wide_dynamic_range_and_special_rows(cuda_device):
    """Rows of very different magnitude, a row whose entries span many orders of magnitude, an
    all-zero row, a denormal-sized row and a row with a NaN: the 22-bit digits follow each row's own
    maximum; a non-finite row gives NaN outputs and does not disturb the token next to it."""
    case = syn.make_case("imma_range", 6, 4096, 256, 4, 128, seed=98, bias=False)
    rng = np.random.default_rng(2)
    case.a[0] *= 1e4
    case.a[1] *= 1e-6
    case.a[2] *= np.exp(rng.uniform(-8, 8, size=case.k)).astype(np.float32)
    case.a[3] = 0.0
    case.a[4] *= 1e-30
    case.a[5, 17] = np.nan
    y, _ = run_device(case, path=_capi.PATH_GEMV_IMMA)
    finite = syn.make_case("imma_range", 6, 4096, 256, 4, 128, seed=98, bias=False)
    finite.a[:5] = case.a[:5]
    ref = oracle_f64(finite)
    for row in (0, 1, 2, 4):   # no bias: tiny rows are compared on their own scale
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    assert not y[3].any()
    assert np.isnan(y[5]).all()


def test_decode_imma_path_rejects_small_blocks(cuda_device):
    import torch

    case = syn.make_case("imma_reject", 1, 4096, 64, 4, 32, seed=8)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=4096, N=64, bits=4, block_size=32)
    with pytest.raises(_capi.MatMulNBitsError) as info:
        weights.matmul_device(torch.from_numpy(case.a).cuda(), torch.zeros((1, 64), device="cuda"),
                              path=_capi.PATH_GEMV_IMMA)
    assert info.value.status == _capi.MNB_ERR_UNSUPPORTED
    weights.close()


# shapes for the direct-stream decode kernel: (m, k, n, zp, bias)
DIRECT_CASES = [
    (1, 4096, 96, True, True),         # one token: eight-row tiles, two segments per step
    (1, 4096, 77, False, False),       # ragged last tile, default zero point
    (1, 2048, 40, True, False),        # few tiles: four warps share a tile
    (1, 1536, 50, True, True),         # twelve blocks per row: the one-token form does not fit, sixteen-row tiles
    (1, 1024, 33, True, False),        # eight blocks per row with zero points: AUTO's choice (no resident form)
    (1, 14336, 48, True, True),        # wide K (down projection)
    (1, 4000, 50, True, True),         # K not a multiple of the block
    (1, 4096, 7, True, True),          # fewer rows than a tile
    (2, 4096, 200, False, True),       # two tokens = one column tile
    (2, 2048, 333, True, False),
    (1, 4096, 14336, True, True),      # cfg2 at full size
    (2, 4096, 14336, False, True),
]


@pytest.mark.parametrize("m,k,n,zp,bias", DIRECT_CASES)
def test_decode_direct_path(cuda_device, m, k, n, zp, bias):
    case = syn.make_case("direct", m, k, n, 4, 128, seed=m * 19 + k + n, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_DIRECT)
    assert kernel == DIRECT
    ref = oracle_f64(case)
    for row in range(m):   # every token against its own magnitude
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    y_auto, kernel_auto = run_device(case)
    if resident_takes(case):
        assert kernel_auto == RESIDENT and rel_err(y, y_auto) <= TOL_FP32
    elif direct_takes(case):
        assert kernel_auto == DIRECT and np.array_equal(y, y_auto)
    else:
        assert rel_err(y, y_auto) <= TOL_FP32


# shapes for the one-token resident decode kernel: (k, n, zp, bias)
RESIDENT_CASES = [
    (4096, 96, True, True),          # one slot per tile, nothing refilled
    (4096, 77, False, False),        # ragged last tile (rows beyond N filled with zeros), default zero point
    (2048, 40, True, False),
    (1024, 50, False, True),         # eight blocks per row
    (14336, 48, True, True),         # wide K: tasks of eight chunks, two slots per warp, seven parts per tile
    (4000, 50, True, True),          # K not a multiple of the block
    (4096, 7, True, True),           # fewer rows than a tile
    (4096, 14336, True, True),       # cfg2 at full size: one slot is refilled on the SMs with thirteen tiles
    (4096, 14336, False, False),
    (4096, 40000, True, False),      # many tiles per SM: every slot refilled several times
    (8192, 4096, True, True),
]


@pytest.mark.parametrize("k,n,zp,bias", RESIDENT_CASES)
def test_decode_resident_path(cuda_device, k, n, zp, bias):
    case = syn.make_case("resident", 1, k, n, 4, 128, seed=k + n, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_RESIDENT)
    assert kernel == RESIDENT
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32
    y_auto, kernel_auto = run_device(case)
    if resident_takes(case):
        assert kernel_auto == RESIDENT and np.array_equal(y, y_auto)
    else:
        assert kernel_auto == DIRECT and rel_err(y, y_auto) <= 1e-6
    y_direct, _ = run_device(case, path=_capi.PATH_GEMV_DIRECT)   # same digits, same block sums
    assert rel_err(y, y_direct) <= 1e-6


# the same kernel with blocks of 32 (one MMA per block): (k, n, zp, bias)
RESIDENT_BLOCK32_CASES = [
    (4096, 96, True, True),          # zero points straight from the operator's packed nibbles
    (4096, 77, False, False),        # ragged last tile, default zero point
    (1024, 50, False, True),         # one chunk of 32 scales per row
    (2048, 8, True, False),          # a single tile
    (3072, 272, True, True),         # three chunks of scales per row
    (8192, 520, False, True),        # wide K: tasks of part of a row
    (4096, 1001, False, False),      # N not a multiple of eight: tile by tile copies
    (4096, 4096, False, False),      # cfg1 at full size
    (4096, 16032, True, False),      # one of eight column shards of the large-N projection
]


@pytest.mark.parametrize("k,n,zp,bias", RESIDENT_BLOCK32_CASES)
def test_decode_resident_path_block32(cuda_device, k, n, zp, bias):
    case = syn.make_case("resident32", 1, k, n, 4, 32, seed=k + n + 32, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_RESIDENT)
    assert kernel == RESIDENT
    if n > 4096:
        columns = np.random.default_rng(7).choice(n, size=512, replace=False)
        ref = o.matmul_f64(case.a, case.b.reshape(n, -1)[columns].reshape(-1), case.scales.reshape(n, -1)[columns].reshape(-1),
                           None if case.zero_points is None else case.zero_points.reshape(n, -1)[columns].reshape(-1),
                           None if case.bias is None else case.bias[columns], len(columns), k, 4, 32)
        assert rel_err(y[:, columns], ref) <= TOL_FP32
    else:
        assert rel_err(y, oracle_f64(case)) <= TOL_FP32
    y_auto, kernel_auto = run_device(case)
    if resident_takes(case):
        assert kernel_auto == RESIDENT and np.array_equal(y, y_auto)
    else:
        assert kernel_auto == "nbits_gemv_mma_kernel"
    y_mma, name = run_device(case, path=_capi.PATH_GEMV_MMA)   # the fp16 two-piece kernel on the same node
    assert name == "nbits_gemv_mma_kernel"
    assert rel_err(y, y_mma) <= TOL_FP32


def test_decode_resident_block32_special_rows(cuda_device):
    for value, expect_nan in ((np.nan, True), (np.inf, True), (0.0, False)):
        case = syn.make_case("resident32_special", 1, 4096, 64, 4, 32, seed=3, bias=True)
        if value == 0.0:
            case.a[:] = 0.0
        else:
            case.a[0, 4000] = value
        y, kernel = run_device(case, path=_capi.PATH_GEMV_RESIDENT)
        assert kernel == RESIDENT
        if expect_nan:
            assert np.isnan(y).all()
        else:
            assert np.array_equal(y[0], case.bias)


def test_decode_resident_path_special_rows_and_rejections(cuda_device):
    import torch

    for value, expect_nan in ((np.nan, True), (np.inf, True), (0.0, False)):
        case = syn.make_case("resident_special", 1, 4096, 64, 4, 128, seed=3, bias=True)
        if value == 0.0:
            case.a[:] = 0.0
        else:
            case.a[0, 4000] = value
        y, kernel = run_device(case, path=_capi.PATH_GEMV_RESIDENT)
        assert kernel == RESIDENT
        if expect_nan:
            assert np.isnan(y).all()
        else:
            assert np.array_equal(y[0], case.bias)
    case = syn.make_case("resident_reject", 2, 4096, 64, 4, 128, seed=8)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=4096, N=64, bits=4, block_size=128)
    with pytest.raises(_capi.MatMulNBitsError) as info:   # two tokens
        weights.matmul_device(torch.from_numpy(case.a).cuda(), torch.zeros((2, 64), device="cuda"),
                              path=_capi.PATH_GEMV_RESIDENT)
    assert info.value.status == _capi.MNB_ERR_UNSUPPORTED
    weights.close()


def test_decode_direct_path_special_rows(cuda_device):
    """Rows of very different magnitude, an all-zero row, a denormal-sized row and a row with a
    NaN: the 22-bit digits follow each row's own maximum; a non-finite row gives NaN outputs and
    does not disturb the tokens next to it."""
    case = syn.make_case("direct_range", 6, 4096, 256, 4, 128, seed=98, bias=False)
    rng = np.random.default_rng(2)
    case.a[0] *= 1e4
    case.a[1] *= 1e-6
    case.a[2] *= np.exp(rng.uniform(-8, 8, size=case.k)).astype(np.float32)
    case.a[3] = 0.0
    case.a[4] *= 1e-30
    case.a[5, 17] = np.nan
    rows = []
    for first in (0, 2, 4):   # the kernel takes two tokens per call
        pair = syn.make_case("direct_range", 2, 4096, 256, 4, 128, seed=98, bias=False)
        pair.b, pair.scales, pair.zero_points = case.b, case.scales, case.zero_points
        pair.a = case.a[first:first + 2].copy()
        y_pair, kernel = run_device(pair, path=_capi.PATH_GEMV_DIRECT)
        assert kernel == DIRECT
        rows.append(y_pair)
    y = np.concatenate(rows)
    finite = syn.make_case("direct_range", 6, 4096, 256, 4, 128, seed=98, bias=False)
    finite.a[:5] = case.a[:5]
    ref = oracle_f64(finite)
    for row in (0, 1, 2, 4):   # no bias: tiny rows are compared on their own scale
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    assert not y[3].any()
    assert np.isnan(y[5]).all()
    one = syn.make_case("direct_nan", 1, 4096, 64, 4, 128, seed=3)
    one.a[0, 4000] = np.inf
    y1, _ = run_device(one, path=_capi.PATH_GEMV_DIRECT)
    assert np.isnan(y1).all()


def test_decode_direct_path_rejects_other_blocks(cuda_device):
    import torch

    case = syn.make_case("direct_reject", 1, 4096, 64, 4, 32, seed=8)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=4096, N=64, bits=4, block_size=32)
    with pytest.raises(_capi.MatMulNBitsError) as info:
        weights.matmul_device(torch.from_numpy(case.a).cuda(), torch.zeros((1, 64), device="cuda"),
                              path=_capi.PATH_GEMV_DIRECT)
    assert info.value.status == _capi.MNB_ERR_UNSUPPORTED
    weights.close()


# shapes for the digit kernels (PATH_GEMV_DIGITS: the one-pass kernel where it fits): (m, k, n, block, zp, bias)
DIGIT_ROW_CASES = [
    (16, 4096, 128, 32, False, True),      # 48 digit rows, two slices, default zero point
    (5, 4096, 77, 64, True, True),         # five tokens: 24 digit rows, nine of them empty
    (3, 2048, 200, 128, True, False),      # three tokens, one slice
    (16, 4096, 300, 128, True, True),
    (1, 4096, 64, 32, True, False),        # three rows: one pass of eight
    (7, 8192, 40, 256, False, False),      # block spans two 128-k table entries
    (11, 14336, 96, 32, True, True),       # wide K: seven slices; 33 rows = three passes, last one ragged
    (16, 4096, 14336, 32, False, False),   # cfg4 gate / up projection at full size
    (16, 1024, 256, 32, False, False),     # K shorter than one 2048-k slice: the rest of the slice is zeros
    (9, 6144, 100, 128, True, True),       # three slices, the SMs do not divide by them
    (12, 4096, 24, 1024, True, False),     # one quantization block spans eight 128-k table entries
]


@pytest.mark.parametrize("m,k,n,bs,zp,bias", DIGIT_ROW_CASES)
def test_decode_digit_rows_path(cuda_device, m, k, n, bs, zp, bias):
    case = syn.make_case("digit_rows", m, k, n, 4, bs, seed=m * 17 + k + n + bs, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_GEMV_DIGITS)
    assert kernel == "nbits_digits_mma_kernel"
    ref = oracle_f64(case)
    for row in range(m):
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    y_auto, kernel_auto = run_device(case)
    assert rel_err(y, y_auto) <= TOL_FP32


def test_decode_digit_rows_special_rows(cuda_device):
    """An all-zero row gives the bias, a row with a NaN gives NaN and leaves its neighbours alone,
    rows of very different magnitude keep their own relative accuracy."""
    case = syn.make_case("digit_rows_special", 6, 4096, 128, 4, 32, seed=97, bias=False)
    case.a[0] *= 1e4
    case.a[1] *= 1e-6
    case.a[2] = 0.0
    case.a[3] *= 1e-30
    case.a[4, 100] = np.nan
    y, _ = run_device(case, path=_capi.PATH_GEMV_DIGITS)
    finite = syn.make_case("digit_rows_special", 6, 4096, 128, 4, 32, seed=97, bias=False)
    finite.a[:4] = case.a[:4]
    ref = oracle_f64(finite)
    for row in (0, 1, 3, 5):
        assert rel_err(y[row], ref[row]) <= TOL_FP32, row
    assert not y[2].any()
    assert np.isnan(y[4]).all()


def test_generic_kernel_matches_stream_kernel(cuda_device):
    """Two independent CUDA implementations of the decode path agree."""
    import torch

    case = syn.make_case("cross", 2, 4096, 513, 4, 32, seed=42, bias=True)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n)
    a = torch.from_numpy(case.a).cuda()
    y1 = torch.empty((2, 513), device="cuda")
    weights.matmul_device(a, y1, path=_capi.PATH_GEMV)
    # block_size 16 is outside what the stream kernel takes, so it runs on the word-wise one
    case2 = syn.make_case("cross", 2, 4096, 513, 4, 16, seed=42, bias=True)
    torch.cuda.synchronize()
    assert _capi.last_kernel().startswith("nbits_gemv_stream")
    y_ref = oracle_f64(case)
    assert rel_err(y1.cpu().numpy(), y_ref) <= TOL_FP32
    y2, kernel2 = run_device(case2)
    assert kernel2 == "nbits_gemv_words_kernel"
    assert rel_err(y2, oracle_f64(case2)) <= TOL_FP32


# Shapes no staged kernel takes: block_size 16, 8-bit rows too long for whole-row stages, K that is
# not a multiple of eight (scalar activation loads), ragged N, more tokens than one pass takes.
WORDS_CASES = [
    # m, k, n, bits, block, zp, bias
    (1, 4096, 515, 4, 16, True, True),
    (2, 1024, 33, 4, 16, False, False),
    (3, 8192, 70, 4, 16, True, False),
    (7, 4096, 129, 4, 16, True, True),
    (16, 2048, 31, 4, 16, False, True),
    (1, 14336, 257, 8, 128, True, True),
    (2, 14336, 64, 8, 512, False, False),
    (4, 14336, 100, 8, 512, True, False),
    (16, 14336, 37, 8, 512, True, True),
    (4, 8192, 50, 8, 16, True, False),
    (20, 1024, 45, 8, 16, True, True),       # three passes of eight tokens
    (40, 512, 19, 4, 16, True, False),       # five passes
    (3, 1003, 21, 4, 16, True, True),        # K odd: scalar activation loads, a partly filled last group
    (18, 72, 5, 8, 16, False, True),         # partial last block
    (9, 14336, 40, 8, 512, True, True),      # a block longer than a chunk of 256 codes
    (19, 264, 300, 8, 16, True, False),      # a last chunk of one group, more columns than one CTA
]


@pytest.mark.parametrize("m,k,n,bs,expected", [
    (2, 4096, 200, 32, "nbits_gemv_stream_kernel"),        # two tokens: one pass of the staged kernel
    (3, 4096, 200, 32, "nbits_gemv_columns_kernel"),       # a narrow node, three and four tokens
    (2, 4096, 5000, 128, "nbits_gemv_stream_kernel"),      # a wide node, two tokens
    (3, 4096, 5000, 128, "nbits_gemv_u8_mma_kernel"),      # a wide node from three tokens on: integer tensor cores
    (5, 4096, 200, 128, "nbits_gemv_u8_mma_kernel"),       # any node from five tokens on
    (16, 8192, 333, 64, "nbits_gemv_u8_mma_kernel"),
    (8, 4096, 200, 512, "nbits_gemv_columns_kernel"),      # blocks the tensor-core kernel does not take
])
def test_eight_bit_decode_kernels_under_auto(cuda_device, m, k, n, bs, expected):
    case = syn.make_case("u8tokens", m, k, n, 8, bs, seed=m + n, zero_points=True, bias=True)
    y, kernel = run_device(case)
    assert kernel.startswith(expected), kernel
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32


# 8-bit weights on integer tensor cores: every block size it takes, with and without zero points and
# bias, one and two column tiles of tokens, ragged N (a last row tile that is partly filled, fewer rows
# than one tile), K that is not a multiple of the block (padding codes meet zero digits), rows long
# enough for several tiles of weights per warp and short enough for less than one.
U8_MMA_CASES = [
    # m, k, n, block, zp, bias
    (5, 4096, 77, 32, True, True),
    (8, 4096, 149, 64, True, False),
    (8, 1024, 300, 128, False, True),
    (9, 8192, 40, 256, True, True),
    (16, 14336, 37, 32, True, True),
    (5, 4000, 33, 32, True, True),
    (16, 4096, 1000, 128, True, False),
    (6, 40, 3, 32, True, True),
    (13, 14336, 260, 128, False, False),
    (7, 96, 16, 32, True, False),
    (16, 2048, 2100, 64, True, True),
    (2, 14336, 64, 32, False, False),        # rows too long for the staged kernel, two tokens
    (4, 14336, 100, 64, True, False),
]


@pytest.mark.parametrize("m,k,n,bs,zp,bias", U8_MMA_CASES)
def test_eight_bit_tensor_core_decode(cuda_device, m, k, n, bs, zp, bias):
    case = syn.make_case("u8mma", m, k, n, 8, bs, seed=3 * m + n, zero_points=zp, bias=bias)
    y, kernel = run_device(case)
    assert kernel == "nbits_gemv_u8_mma_kernel", kernel
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32
    assert rel_err(y, o.matmul_f32(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 8, bs)) <= TOL_FP32


def test_eight_bit_tensor_core_decode_special_rows(cuda_device):
    """A token of zeros gives the bias; a NaN in a token reaches all of that token's outputs and no other;
    a token 2^40 times larger than the others keeps its relative error (each token has its own factor)."""
    case = syn.make_case("u8rows", 6, 1024, 70, 8, 64, seed=11, zero_points=True, bias=True)
    case.a[1] = 0.0
    case.a[3, 17] = np.nan
    case.a[4] *= np.float32(2.0 ** 40)
    case.a[5] *= np.float32(2.0 ** -110)
    y, kernel = run_device(case)
    assert kernel == "nbits_gemv_u8_mma_kernel", kernel
    assert np.array_equal(y[1], case.bias)
    assert np.isnan(y[3]).all()
    ref = oracle_f64(case)
    for token in (0, 2, 4):
        assert rel_err(y[token], ref[token]) <= TOL_FP32, token
    assert not np.isnan(y[5]).any()
    assert np.abs(y[5] - case.bias).max() <= 1e-20


@pytest.mark.parametrize("m,k,n,bits,bs,zp,bias", WORDS_CASES)
def test_word_wise_kernel(cuda_device, m, k, n, bits, bs, zp, bias):
    case = syn.make_case("words", m, k, n, bits, bs, seed=m * 31 + n, zero_points=zp, bias=bias)
    y, kernel = run_device(case)
    # lanes along K for one and two tokens, a lane per output column from three tokens on
    assert kernel == ("nbits_gemv_words_kernel" if m <= 2 else "nbits_gemv_columns_kernel"), kernel
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32


def test_strided_output_window(cuda_device):
    import torch

    case = syn.make_case("win", 2, 4096, 64, 4, 32, seed=8, bias=True)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n)
    y = torch.zeros((2, 200), device="cuda")
    weights.matmul_device(torch.from_numpy(case.a).cuda(), y, ld_y=200, col_offset=100)
    torch.cuda.synchronize()
    out = y.cpu().numpy()
    assert not out[:, :100].any() and not out[:, 164:].any()
    assert rel_err(out[:, 100:164], oracle_f64(case)) <= TOL_FP32


def test_decode_linearity_at_full_size(cuda_device):
    """Size-independent property on the full cfg2 shape: f(a1 + a2) = f(a1) + f(a2) - f(0)."""
    base = syn.config2(1)
    rng = np.random.default_rng(5)
    a1 = rng.standard_normal((1, base.k)).astype(np.float32)
    a2 = rng.standard_normal((1, base.k)).astype(np.float32)
    outs = []
    for a in (a1, a2, a1 + a2, np.zeros_like(a1)):
        base.a = a
        outs.append(run_device(base)[0].astype(np.float64))
    lhs = outs[2]
    rhs = outs[0] + outs[1] - outs[3]
    assert np.abs(lhs - rhs).max() / np.abs(lhs).max() <= 2e-5
    assert np.allclose(outs[3][0], base.bias, rtol=0, atol=0)  # zero activations leave the bias


# ---- prefill path (bf16 tcgen05) -------------------------------------------------------------------
@pytest.mark.parametrize("m,k,n,bs,zp,bias", [
    (512, 4096, 512, 64, True, False),     # cfg3 geometry at reduced N
    (64, 1024, 128, 32, True, True),
    (200, 2048, 300, 128, False, True),    # ragged M and N
    (17, 256, 130, 64, True, False),
    (256, 512, 128, 256, True, True),
    (300, 4096, 256, 64, True, False),
])
def test_prefill_tcgen05(cuda_device, m, k, n, bs, zp, bias):
    case = syn.make_case("prefill", m, k, n, 4, bs, seed=m + k + n, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_TCGEN05)
    expected = "nbits_gemm_tcgen05_kernel"   # few tiles: 128-row tiles
    assert kernel.startswith(expected), kernel
    ref_bf16 = o.matmul_bf16(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 4, bs)
    assert rel_err(y, ref_bf16) <= TOL_BF16
    assert rel_err(y, oracle_f64(case)) <= TOL_BF16


@pytest.mark.parametrize("m,k,n,bs,zp,bias", [
    (17, 256, 130, 64, True, False),       # 64-token tile, ragged N
    (64, 1024, 128, 32, True, True),
    (100, 2048, 300, 128, False, True),    # 128-token tile, default zero point 128
    (300, 4096, 256, 32, True, False),     # 256-token tile
    (256, 4096, 1002, 32, True, False),    # the column-shard geometry at reduced N
])
def test_prefill_tcgen05_8bit(cuda_device, m, k, n, bs, zp, bias):
    """8-bit codes through the same kernel: whole bytes, natural k order, (q - zp) exact in bf16."""
    case = syn.make_case("prefill8", m, k, n, 8, bs, seed=m + k + n + 8, zero_points=zp, bias=bias)
    y, kernel = run_device(case)   # AUTO: above sixteen tokens 8-bit weights go to the tensor cores too
    assert kernel.startswith("nbits_gemm_tcgen05"), kernel
    ref_bf16 = o.matmul_bf16(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 8, bs)
    assert rel_err(y, ref_bf16) <= TOL_BF16
    assert rel_err(y, oracle_f64(case)) <= TOL_BF16


PAIR = "nbits_gemm_tcgen05_pair_kernel"


@pytest.mark.parametrize("m,k,n,bs,zp,bias", [
    (300, 4096, 700, 32, True, True),      # ragged in both directions, zero points as whole bytes
    (64, 1024, 128, 64, False, False),     # default zero point 128, a single pair
    (256, 4096, 1002, 32, True, False),    # the column-shard geometry at reduced N
])
def test_prefill_tcgen05_cta_pairs_8bit(cuda_device, m, k, n, bs, zp, bias):
    """8-bit codes through the pair kernel: 64 packed bytes per row and k step, natural k order."""
    case = syn.make_case("prefill_pair8", m, k, n, 8, bs, seed=m + k + n + 88, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_TCGEN05_WIDE)
    assert kernel.startswith(PAIR), kernel
    rows, name = run_device(case, path=_capi.PATH_TCGEN05)
    assert name.startswith("nbits_gemm_tcgen05_kernel"), name
    ref_bf16 = o.matmul_bf16(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 8, bs)
    assert rel_err(y, ref_bf16) <= TOL_BF16
    assert rel_err(y, oracle_f64(case)) <= TOL_BF16
    assert rel_err(y, rows) <= 1e-5        # the same roundings as the 128-row kernel, another order of the fp32 sums


@pytest.mark.parametrize("m,k,n,bs,zp,bias", [
    (512, 4096, 512, 64, True, False),
    (300, 1024, 700, 32, True, True),      # ragged in both directions; the odd CTA's second sub-tile is past N
    (257, 512, 130, 128, False, True),     # one token over a tile boundary; the odd CTA of the pair has no row at all
    (64, 256, 256, 64, True, False),
    (1024, 1024, 1536, 64, True, True),    # three pairs of row tiles, K whole
    (250, 2048, 1000, 32, True, True),     # token tile narrower than 256 and not a multiple of 32
    (17, 4096, 520, 64, True, True),       # fewer tokens than the narrowest tile, K in eight parts
    (40, 14336, 300, 32, False, False),    # 224 k steps in eight parts of 28
])
def test_prefill_tcgen05_cta_pairs(cuda_device, m, k, n, bs, zp, bias):
    """The kernel in which two CTAs share every MMA (each with 256 weight rows of its own and half of
    the token tile), forced for shapes of every raggedness; K whole or shared between pairs as the
    plan decides."""
    case = syn.make_case("prefill_pair", m, k, n, 4, bs, seed=m + k + n + 1, zero_points=zp, bias=bias)
    y, kernel = run_device(case, path=_capi.PATH_TCGEN05_WIDE)
    assert kernel.startswith(PAIR), kernel
    ref_bf16 = o.matmul_bf16(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 4, bs)
    assert rel_err(y, ref_bf16) <= TOL_BF16
    assert rel_err(y, oracle_f64(case)) <= TOL_BF16


@pytest.mark.parametrize("m,k,n,bs,zp,bias", [
    (200, 4096, 4100, 64, True, True),     # nine pairs of row tiles (the last one ragged), K in four parts
    (256, 4096, 4096, 32, True, False),
    (64, 4096, 4096, 64, True, True),      # the middle regime on a square node: AUTO shares K between pairs
])
def test_prefill_split_k(cuda_device, m, k, n, bs, zp, bias):
    """Products between decode and prefill whose tiles alone would leave most SMs idle: K is shared
    by several CTA pairs per tile and the partial products are added in part order by a kernel
    behind them, so two runs give the same bits. Values match the bf16 model like the 128-row
    kernel's, and that kernel itself up to the order of the fp32 additions."""
    case = syn.make_case("splitk", m, k, n, 4, bs, seed=m + k + n + 5, zero_points=zp, bias=bias)
    y, kernel = run_device(case)
    again, _ = run_device(case)
    assert kernel == PAIR + "(split-k)", kernel
    np.testing.assert_array_equal(y, again)
    ref_bf16 = o.matmul_bf16(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 4, bs)
    assert rel_err(y, ref_bf16) <= TOL_BF16
    assert rel_err(y, oracle_f64(case)) <= TOL_BF16
    whole, name = run_device(case, path=_capi.PATH_TCGEN05)
    assert name.startswith("nbits_gemm_tcgen05_kernel"), name
    assert rel_err(y, whole) <= 1e-5


def test_four_tokens_on_long_rows_stay_on_tensor_cores(cuda_device):
    """M = 4, block 128, K = 14336: the fp16 kernels cannot stage four tokens of that length, and the
    product used to fall through to the scalar kernel (1.8 ms for the square node). AUTO takes the
    one-pass digit kernel from three tokens on for rows of 8192 k and more."""
    for m in (3, 4):
        case = syn.make_case("long_rows", m, 14336, 264, 4, 128, seed=77 + m, zero_points=True, bias=True)
        y, kernel = run_device(case)
        assert kernel == SLICED, kernel
        assert rel_err(y, oracle_f64(case)) <= TOL_FP32


def test_prefill_kernels_agree_on_random_shapes(cuda_device):
    """Forty seeded random shapes (4- and 8-bit, every block size, ragged M and N, 17 to 3000 tokens):
    the pair kernel, whatever AUTO picks, and the 128-row kernel round the same way, so whole-K
    products agree bit for bit and products with K shared between pairs up to the order of the
    fp32 additions."""
    rng = np.random.default_rng(20260)
    for it in range(40):
        bits = int(rng.choice([4, 4, 4, 8]))
        bs = int(rng.choice([32, 64, 128, 256]))
        k = int(rng.integers(1, 40)) * 64
        k = -(-k // bs) * bs
        n = int(rng.integers(1, 1400)) if rng.random() < 0.7 else int(rng.integers(1, 9)) * 512 + int(rng.integers(-3, 4))
        m = int(rng.integers(17, 700)) if rng.random() < 0.8 else int(rng.integers(700, 3000))
        zp, bias = bool(rng.integers(0, 2)), bool(rng.integers(0, 2))
        case = syn.make_case("prefill_random", m, k, n, bits, bs, seed=3000 + it, zero_points=zp, bias=bias)
        rows, name = run_device(case, path=_capi.PATH_TCGEN05)
        assert name.startswith("nbits_gemm_tcgen05_kernel"), name
        scale = float(np.abs(rows).max()) + 1e-30
        for path in (_capi.PATH_TCGEN05_WIDE, _capi.PATH_AUTO):
            y, kernel = run_device(case, path=path)
            assert kernel.startswith("nbits_gemm_tcgen05"), kernel
            assert not np.isnan(y).any(), (it, kernel)
            tolerance = 2e-5 if kernel.endswith("(split-k)") else 0.0
            assert float(np.abs(y - rows).max()) / scale <= tolerance, (it, m, k, n, bits, bs, kernel)


def test_prefill_auto_dispatch_and_full_size_property(cuda_device):
    """cfg3 at full size M=2048: a checksum identity instead of a full CPU product. With A = ones
    the result is the per-column sum of the (bf16-rounded) dequantized weights."""
    import torch

    case = syn.config3(2048)
    case.a = np.ones_like(case.a)
    y, kernel = run_device(case)
    assert kernel.startswith("nbits_gemm_tcgen05"), kernel
    ints = o.dequant_int(case.b, case.zero_points, case.n, case.k, 4, 64).astype(np.float64)
    scales = np.repeat(case.scales.reshape(case.n, -1).astype(np.float64), 64, axis=1)
    col_sums = (ints * scales).sum(axis=1)
    assert np.abs(y - y[0:1]).max() == 0.0                     # all rows identical
    assert rel_err(y[0], col_sums) <= TOL_BF16


# ---- accuracy_level 4 ----------------------------------------------------------------------------------
@pytest.mark.parametrize("m,k,bs", [(16, 4096, 32), (3, 200, 64), (1, 4096, 128), (5, 48, 16)])
def test_activation_quantization_bit_exact(cuda_device, m, k, bs):
    import torch

    rng = np.random.default_rng(m + k)
    a = rng.standard_normal((m, k)).astype(np.float32)
    a[0, :bs] = 0.0
    nb = -(-k // bs)
    aq = torch.empty((m, k), dtype=torch.int8, device="cuda")
    sa = torch.empty((m, nb), dtype=torch.float32, device="cuda")
    quantize_a(torch.from_numpy(a).cuda(), aq, sa, bs)
    torch.cuda.synchronize()
    ref_q, ref_s = o.quantize_a(a, k, bs)
    assert np.array_equal(sa.cpu().numpy(), ref_s)
    assert np.array_equal(aq.cpu().numpy(), ref_q)


@pytest.mark.parametrize("bits,bs,k,n", [(4, 32, 4096, 40), (4, 128, 512, 9), (8, 32, 256, 17), (4, 16, 80, 5)])
def test_int8_block_dots_bit_exact(cuda_device, bits, bs, k, n):
    import torch

    case = syn.make_case("dots", 4, k, n, bits, bs, seed=bits + bs + k)
    aq, _ = o.quantize_a(case.a, k, bs)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, None, K=k, N=n, bits=bits, block_size=bs)
    dots = torch.empty((4, n, case.n_blocks), dtype=torch.int32, device="cuda")
    weights.int8_block_dots(torch.from_numpy(aq).cuda(), dots)
    torch.cuda.synchronize()
    assert np.array_equal(dots.cpu().numpy(), o.int8_block_dots(aq, case.b, case.zero_points, n, k, bits, bs))


@pytest.mark.parametrize("m,k,n,bits,bs,zp", [(5, 80, 7, 4, 16, True), (16, 4096, 33, 4, 16, False),
                                              (20, 1000, 12, 4, 16, True), (3, 72, 5, 8, 16, True)])
def test_int8_path_block16(cuda_device, m, k, n, bits, bs, zp):
    """accuracy_level 4 under AUTO with blocks of sixteen: groups of eight codes for 4-bit weights."""
    case = syn.make_case("lvl4b16", m, k, n, bits, bs, seed=m + n, zero_points=zp, bias=True)
    y, kernel = run_device(case, accuracy_level=4)
    assert kernel == ("nbits_int8_words_kernel<4>" if bits == 4 else "nbits_int8_matmul_kernel<8>"), kernel
    ref = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, bits, bs)
    assert rel_err(y, ref) <= TOL_FP32
    assert rel_err(y, oracle_f64(case)) <= 3e-2   # int8 activations vs exact


@pytest.mark.parametrize("m,k,n,bs,zp", [(16, 4096, 200, 32, True), (8, 1024, 50, 64, False), (5, 4000, 33, 32, True),
                                         (9, 14336, 40, 128, True), (1, 4096, 77, 256, True), (3, 96, 7, 32, True)])
def test_int8_path_eight_bit_weights_on_integer_mma(cuda_device, m, k, n, bs, zp):
    """accuracy_level 4 under AUTO with 8-bit weights: the quantized activations as MMA columns."""
    case = syn.make_case("lvl4u8", m, k, n, 8, bs, seed=2 * m + n, zero_points=zp, bias=True)
    y, kernel = run_device(case, accuracy_level=4)
    assert kernel == "nbits_gemv_u8_int8_mma_kernel", kernel
    ref = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 8, bs)
    assert rel_err(y, ref) <= TOL_FP32   # same integers, fp32 scaling in a different order
    assert rel_err(y, oracle_f64(case)) <= 3e-2   # int8 activations vs exact


@pytest.mark.parametrize("m,k,n,bits,bs,zp", [(16, 4096, 128, 4, 32, False), (1, 4096, 77, 4, 128, True),
                                              (9, 1024, 50, 8, 32, True), (16, 4064, 31, 4, 32, True)])
def test_int8_path_outputs(cuda_device, m, k, n, bits, bs, zp):
    case = syn.make_case("lvl4", m, k, n, bits, bs, seed=m + n, zero_points=zp, bias=True)
    y, kernel = run_device(case, accuracy_level=4, path=_capi.PATH_INT8)
    assert kernel.startswith("nbits_int8_matmul_kernel"), kernel
    ref = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, bits, bs)
    assert rel_err(y, ref) <= TOL_FP32   # same integers, fp32 scaling in a different order
    assert rel_err(y, oracle_f64(case)) <= 2e-2   # int8 activations vs exact


# integer tensor-core kernel: every block size class, with and without zero points, one and two
# column tiles of tokens, several passes, ragged N, a last task that is only partly filled, a K
# that ends inside a block, and a K long enough to need the 8-token layout
@pytest.mark.parametrize("m,k,n,bs,zp,bias", [
    (16, 4096, 128, 32, False, True), (16, 4096, 100, 32, True, True), (1, 4096, 77, 128, True, False),
    (8, 2048, 48, 64, True, True), (5, 2304, 33, 64, False, False), (16, 4096, 64, 256, True, True),
    (3, 4096, 24, 1024, False, True), (20, 6144, 40, 128, True, True), (37, 2048, 16, 32, True, False),
    (16, 14336, 40, 32, False, True), (9, 2000, 21, 128, True, True), (16, 4096, 2400, 32, False, False),
    (4, 1056, 16, 32, True, True),
])
def test_int8_mma_path_outputs(cuda_device, m, k, n, bs, zp, bias):
    if (((k + bs - 1) // bs) * bs // 2) % 128 != 0:
        # packed rows must be whole 128-byte segments; other shapes go to the dp4a kernel
        case = syn.make_case("imma_fallback", m, k, n, 4, bs, seed=m + n + bs, zero_points=zp, bias=bias)
        y, kernel = run_device(case, accuracy_level=4)
        assert kernel.startswith("nbits_int8_matmul_kernel"), kernel
    else:
        case = syn.make_case("imma", m, k, n, 4, bs, seed=m + n + bs, zero_points=zp, bias=bias)
        y, kernel = run_device(case, accuracy_level=4)
        assert kernel == "nbits_int8_mma_kernel", kernel
        y2, kernel2 = run_device(case, accuracy_level=4, path=_capi.PATH_INT8_MMA)
        assert kernel2 == kernel and np.array_equal(y, y2)   # deterministic
    ref = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, n, k, 4, bs)
    assert rel_err(y, ref) <= TOL_FP32
    assert rel_err(y, oracle_f64(case)) <= 2e-2


def test_int8_mma_path_rejects_unsupported_shapes(cuda_device):
    import torch

    case = syn.make_case("imma_reject", 2, 96, 8, 4, 32, seed=5)   # 48-byte rows
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=96, N=8, bits=4, block_size=32)
    with pytest.raises(_capi.MatMulNBitsError) as info:
        weights.matmul_device(torch.from_numpy(case.a).cuda(), torch.zeros((2, 8), device="cuda"),
                              accuracy_level=4, path=_capi.PATH_INT8_MMA)
    assert info.value.status == _capi.MNB_ERR_UNSUPPORTED
    weights.close()


# ---- through the registered operator (host tensors) -----------------------------------------------
def test_registered_operator_end_to_end(cuda_device):
    pkg.register_kernels()
    pkg.clear_used_kernel_names()
    case = syn.config2(4, n=1024)
    session = pkg.MatMulNBitsSession(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n, bits=4,
                                     block_size=128)
    y = session.run(case.a)
    assert y.shape == (4, 1024)
    assert rel_err(y, oracle_f64(case)) <= TOL_FP32
    assert session.last_device_kernel == "nbits_gemv_mma_kernel"
    y3 = session.run(case.a.reshape(2, 2, case.k))          # leading dims are kept
    assert y3.shape == (2, 2, 1024) and np.array_equal(y3.reshape(4, 1024), y)
    assert pkg.used_kernel_names() == ["onnx_light_cuda::MatMulNBits"] * 2
    big = syn.make_case("op_prefill", 96, 1024, 256, 4, 64, seed=2)
    s2 = pkg.MatMulNBitsSession(big.b, big.scales, big.zero_points, None, K=1024, N=256, bits=4, block_size=64)
    assert rel_err(s2.run(big.a), oracle_f64(big)) <= TOL_BF16
    assert s2.last_device_kernel.startswith("nbits_gemm_tcgen05_kernel")
    s4 = pkg.MatMulNBitsSession(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n, bits=4,
                                block_size=128, accuracy_level=4)
    ref4 = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 128)
    assert rel_err(s4.run(case.a), ref4) <= TOL_FP32


def test_host_call_pinned_and_pageable_buffers(cuda_device):
    """The host-buffer entry point stores into page-locked result buffers directly and stages any other
    buffer through device memory: both give the device result, call after call."""
    import torch

    case = syn.config2(3, n=1000)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n,
                                     bits=4, block_size=128)
    ref = oracle_f64(case)
    a_pinned = torch.from_numpy(case.a).pin_memory()
    y_pinned = torch.full((3, case.n), float("nan")).pin_memory()
    y_pageable = np.full((3, case.n), np.nan, dtype=np.float32)
    for _ in range(2):
        weights.matmul_host_ptr(a_pinned.data_ptr(), 3, y_pinned.data_ptr())
        assert rel_err(y_pinned.numpy(), ref) <= TOL_FP32
        weights.matmul_host_ptr(case.a.ctypes.data, 3, y_pageable.ctypes.data)
        assert np.array_equal(y_pageable, y_pinned.numpy())
        y_pinned.fill_(float("nan"))
        y_pageable.fill(np.nan)
    # a window of a larger pinned buffer, not 16-byte aligned
    wide = torch.full((3 * case.n + 5,), float("nan")).pin_memory()
    weights.matmul_host_ptr(a_pinned.data_ptr(), 3, wide.data_ptr() + 4 * 3)
    assert rel_err(wide.numpy()[3:3 + 3 * case.n].reshape(3, case.n), ref) <= TOL_FP32
    assert np.isnan(wide.numpy()[:3]).all() and np.isnan(wide.numpy()[3 + 3 * case.n:]).all()
    weights.close()


def test_device_entry_point_refuses_host_pointers(cuda_device):
    import torch

    case = syn.make_case("host_ptr", 1, 4096, 64, 4, 128, seed=3)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, None, None, K=4096, N=64, bits=4, block_size=128)
    y = torch.zeros((1, 64), device="cuda")
    with pytest.raises(_capi.MatMulNBitsError, match="take device memory") as info:
        _capi.check(weights._lib.mnb_matmul_device(weights._handle, case.a.ctypes.data, 1, 0, 0, y.data_ptr(), None))
    assert info.value.status == _capi.MNB_ERR_INVALID_ARGUMENT
    weights.close()


def test_llama_layer_shapes_both_accuracy_levels(cuda_device):
    """cfg4 geometry (seven projections, M=16, block 32, no zero points) at reduced N."""
    for level in (0, 4):
        for full in syn.config4(level):
            n = min(full.n, 256)
            case = syn.make_case(full.name, 16, full.k, n, 4, 32, seed=full.meta["seed"], zero_points=False)
            y, _ = run_device(case, accuracy_level=level)
            if level == 0:
                assert rel_err(y, oracle_f64(case)) <= TOL_FP32
            else:
                ref = o.matmul_int8(case.a, case.b, case.scales, None, None, n, case.k, 4, 32)
                assert rel_err(y, ref) <= TOL_FP32


# ---- the production integer-MMA kernel's own block dots: bit-exact --------------------------------
@pytest.mark.parametrize("m,k,n,bs,zp", [
    (8, 4096, 96, 32, True), (8, 4096, 50, 32, False), (5, 2048, 77, 64, True), (3, 2304, 33, 64, False),
    (8, 4096, 64, 128, True), (1, 4096, 40, 128, False), (7, 4096, 24, 256, True), (2, 4096, 16, 1024, False),
    (4, 2000, 21, 128, True),      # K ends inside a block
])
def test_int8_mma_kernel_block_dots_bit_exact(cuda_device, m, k, n, bs, zp):
    """The instrumented instantiation of nbits_int8_mma_kernel stores every block sum before it is
    scaled: same fragment layout, swizzled tiles, signed-code form (no zero points) and zero-point
    correction as the production kernel. Bit-exact against the CPU restatement, whose int32 dots
    are themselves pinned to the reference's IntegerMatMul2D."""
    import torch

    case = syn.make_case("mma_dots", m, k, n, 4, bs, seed=m + k + n + bs, zero_points=zp, bias=True)
    weights = pkg.MatMulNBitsWeights(case.b, case.scales, case.zero_points, case.bias, K=k, N=n, bits=4, block_size=bs)
    a = torch.from_numpy(case.a).cuda()
    y = torch.empty((m, n), device="cuda")
    dots = torch.full((m, n, case.n_blocks), 12345, dtype=torch.int32, device="cuda")
    weights.int8_mma_block_dots(a, y, dots)
    torch.cuda.synchronize()
    assert weights.poll_status() == 0 and _capi.last_kernel() == "nbits_int8_mma_kernel"
    aq, _ = o.quantize_a(case.a, k, bs)
    assert np.array_equal(dots.cpu().numpy(), o.int8_block_dots(aq, case.b, case.zero_points, n, k, 4, bs))
    # and the instrumented run gives the ordinary result
    y_plain = torch.empty((m, n), device="cuda")
    weights.matmul_device(a, y_plain, accuracy_level=4, path=_capi.PATH_INT8_MMA)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), y_plain.cpu().numpy())
    weights.close()


def test_int8_paths_non_finite_activations(cuda_device):
    """accuracy_level 4: a NaN or an infinity in A gives NaN for every output of that token (scale
    NaN, codes 0) on both kernels and in the CPU restatement; the other tokens are untouched."""
    import torch

    case = syn.make_case("lvl4_nan", 4, 4096, 64, 4, 32, seed=21, bias=True)
    clean = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, 64, 4096, 4, 32)
    case.a[1, 100] = np.nan
    case.a[3, 4000] = -np.inf
    ref = o.matmul_int8(case.a, case.b, case.scales, case.zero_points, case.bias, 64, 4096, 4, 32)
    assert np.isnan(ref[1]).all() and np.isnan(ref[3]).all()
    assert np.array_equal(ref[0], clean[0]) and np.array_equal(ref[2], clean[2])
    aq, sa = o.quantize_a(case.a, 4096, 32)
    assert np.isnan(sa[1, 100 // 32]) and np.isnan(sa[3, 4000 // 32]) and not aq[1, 96:128].any()
    for path in (_capi.PATH_INT8_MMA, _capi.PATH_INT8):
        y, _ = run_device(case, accuracy_level=4, path=path)
        assert np.isnan(y[1]).all() and np.isnan(y[3]).all()
        assert rel_err(y[0], clean[0]) <= TOL_FP32 and rel_err(y[2], clean[2]) <= TOL_FP32
    aq_dev = torch.empty((4, 4096), dtype=torch.int8, device="cuda")
    sa_dev = torch.empty((4, 128), device="cuda")
    quantize_a(torch.from_numpy(case.a).cuda(), aq_dev, sa_dev, 32)
    torch.cuda.synchronize()
    assert np.array_equal(aq_dev.cpu().numpy(), aq)
    assert np.array_equal(sa_dev.cpu().numpy(), sa, equal_nan=True)


def test_registered_operator_notices_rewritten_weights(cuda_device):
    """The per-node cache of uploaded constants is keyed on a fingerprint of their contents too: an
    initializer rewritten in place (same address, other bytes) is uploaded again."""
    pkg.register_kernels()
    case = syn.make_case("cache", 2, 1024, 96, 4, 32, seed=5, bias=True)
    session = pkg.MatMulNBitsSession(case.b, case.scales, case.zero_points, case.bias, K=case.k, N=case.n, bits=4,
                                     block_size=32)
    y1 = session.run(case.a)
    assert rel_err(y1, oracle_f64(case)) <= TOL_FP32
    other = syn.make_case("cache", 2, 1024, 96, 4, 32, seed=6, bias=True)
    session.overwrite_b(other.b)
    y2 = session.run(case.a)
    ref2 = o.matmul_f64(case.a, other.b, case.scales, case.zero_points, case.bias, case.n, case.k, 4, 32)
    assert rel_err(y2, ref2) <= TOL_FP32 and rel_err(y2, y1) > 1e-2
    assert np.array_equal(session.run(case.a), y2)   # unchanged weights: the cached upload is used
