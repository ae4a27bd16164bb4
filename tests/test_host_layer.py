"""Host-side contract of the operator class and registration layer (no GPU needed): mirrors
the reference's registration and wrapper tests
(unittests/cc/test_onnx_light_kernel_registration.cc, ..._integer_matmul_kernel.cc:113-126)."""

import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

import onnx_light_cpu_b200 as pkg
from onnx_light_cpu_b200 import _capi, _register

ROOT = Path(__file__).resolve().parent.parent


def test_inventory_is_exact_and_does_not_touch_dispatch_table():
    lib = _register._host_lib()
    before = lib.olc_dispatch_table_size()
    records = pkg.registered_kernels()
    assert lib.olc_dispatch_table_size() == before
    assert [(r.domain, r.op_type, r.device, r.kernel_name, r.types) for r in records] == [
        ("com.microsoft", "MatMulNBits", "CPU", "onnx_light_cuda::MatMulNBits", (1,))]
    assert pkg.registered_kernel_names() == {"MatMulNBits": "onnx_light_cuda::MatMulNBits"}


def test_register_is_idempotent_and_installs_the_key():
    lib = _register._host_lib()
    marker = object()
    assert pkg.register_kernels(marker) is marker
    size = lib.olc_dispatch_table_size()
    pkg.register_kernels()
    assert lib.olc_dispatch_table_size() == size
    assert lib.olc_dispatch_table_has(b"com.microsoft:MatMulNBits") == 1
    assert lib.olc_dispatch_table_has(b"ai.onnx:MatMulNBits") == 0


def test_duplicate_registration_in_one_pass_is_rejected():
    assert _register._host_lib().olc_duplicate_registration_is_rejected() == 1


def _session(**overrides):
    pkg.register_kernels()
    k, n, bs = 64, 4, 32
    args = dict(b=np.zeros((n, 2, 16), np.uint8), scales=np.ones(n * 2, np.float32), K=k, N=n, bits=4, block_size=bs)
    args.update(overrides)
    return pkg.MatMulNBitsSession(**args)


@pytest.mark.parametrize("overrides,a_shape,fragment", [
    (dict(bits=3), (1, 64), "bits must be 4 or 8"),
    (dict(block_size=24), (1, 64), "power of two"),
    (dict(block_size=8), (1, 64), "power of two"),
    (dict(accuracy_level=2), (1, 64), "accuracy_level"),
    (dict(), (1, 63), "last dimension of A"),
    (dict(scales=np.ones(7, np.float32)), (1, 64), "scales must hold"),
    (dict(b=np.zeros(100, np.uint8)), (1, 64), "B must hold"),
    (dict(zero_points=np.zeros((4, 2), np.uint8)), (1, 64), "zero_points must hold"),
    (dict(bias=np.zeros(3, np.float32)), (1, 64), "bias must hold"),
    (dict(_with_g_idx=True), (1, 64), "g_idx"),
])
def test_contract_violations_raise_invalid_argument(overrides, a_shape, fragment):
    session = _session(**overrides)
    with pytest.raises(ValueError, match=fragment):
        session.run(np.zeros(a_shape, np.float32))


def test_usage_log_records_runs_and_can_be_switched_off():
    pkg.clear_used_kernel_names()
    session = _session(bits=3)
    for _ in range(2):
        with pytest.raises(ValueError):
            session.run(np.zeros((1, 64), np.float32))
    assert pkg.used_kernel_names() == ["onnx_light_cuda::MatMulNBits"] * 2
    pkg.set_kernel_usage_recording(False)
    with pytest.raises(ValueError):
        session.run(np.zeros((1, 64), np.float32))
    pkg.set_kernel_usage_recording(True)
    assert len(pkg.used_kernel_names()) == 2
    pkg.clear_used_kernel_names()
    assert pkg.used_kernel_names() == []


def test_empty_batch_needs_no_device():
    y = _session().run(np.zeros((0, 64), np.float32))
    assert y.shape == (0, 4)


def test_c_abi_exports_every_declared_symbol():
    header = (ROOT / "include" / "matmulnbits_b200.h").read_text()
    declared = set(re.findall(r"\b(mnb_[a-z0-9_]+)\s*\(", header))
    assert declared == set(_capi.EXPORTED_SYMBOLS)
    lib = _capi.load()
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.mnb_version().startswith(b"matmulnbits_b200")
    assert _capi.algorithmic_bytes(1, 14336, 4096, 4, 128, True, True) == 31555584
    assert _capi.algorithmic_bytes(1, 4096, 4096, 4, 32, False, False) == 10518528
    assert _capi.algorithmic_bytes(1, 128256, 4096, 4, 32, True, False) == 337073152


def test_c_abi_argument_errors_without_device():
    lib = _capi.load()
    handle = ctypes.c_void_p()
    b = np.zeros(64, np.uint8)
    s = np.ones(4, np.float32)
    rc = lib.mnb_weights_create(0, b.ctypes.data, s.ctypes.data, None, None, 4, 64, 5, 32, ctypes.byref(handle))
    assert rc == _capi.MNB_ERR_INVALID_ARGUMENT and b"bits" in lib.mnb_last_error()
    rc = lib.mnb_weights_create(0, None, s.ctypes.data, None, None, 4, 64, 4, 32, ctypes.byref(handle))
    assert rc == _capi.MNB_ERR_INVALID_ARGUMENT
    assert lib.mnb_matmul_host(None, None, 1, 0, 0, None) == _capi.MNB_ERR_INVALID_ARGUMENT
    if _capi.device_count() == 0:
        rc = lib.mnb_weights_create(0, b.ctypes.data, s.ctypes.data, None, None, 4, 64, 4, 32, ctypes.byref(handle))
        assert rc == _capi.MNB_ERR_CUDA and b"no CPU path" in lib.mnb_last_error()
        with pytest.raises(RuntimeError, match="no CUDA device"):
            _session().run(np.zeros((1, 64), np.float32))


def test_path_and_status_constants_match_the_header():
    """The Python constants are the header's enum values (a selector that drifted would silently pick
    another kernel)."""
    import re
    from pathlib import Path

    from onnx_light_cpu_b200 import _capi

    header = (Path(__file__).resolve().parents[1] / "include" / "matmulnbits_b200.h").read_text()
    paths = dict(re.findall(r"\bMNB_(PATH_[A-Z0-9_]+)\s*=\s*(\d+)", header))
    assert len(paths) >= 10
    for name, value in paths.items():
        assert getattr(_capi, name) == int(value), name
    for name, value in re.findall(r"\b(MNB_(?:OK|ERR_[A-Z_]+))\s*=\s*(-?\d+)", header):
        if hasattr(_capi, name):
            assert getattr(_capi, name) == int(value), name


def test_device_tensor_checks_reject_bad_arguments():
    """The Python layer refuses tensors that would turn into out-of-bounds device accesses behind
    the C ABI (wrong dtype, host memory, too small, strided, wrong GPU). Needs no GPU: the checks
    look at tensor metadata only."""
    import types

    import pytest
    import torch

    from onnx_light_cpu_b200.matmul_nbits import _check_device_tensor

    def fake(dtype=torch.float32, cuda=True, contiguous=True, index=0, numel=16):
        return types.SimpleNamespace(is_cuda=cuda, dtype=dtype, is_contiguous=lambda: contiguous,
                                     device=types.SimpleNamespace(index=index), numel=lambda: numel)

    _check_device_tensor("a", fake(), "float32", 0, 16)
    for bad, match in ((fake(cuda=False), "CUDA tensor"), (fake(dtype=torch.float16), "dtype float32"),
                       (fake(contiguous=False), "contiguous"), (fake(index=1), "GPU 1"), (fake(numel=8), "are needed")):
        with pytest.raises(ValueError, match=match):
            _check_device_tensor("a", bad, "float32", 0, 16)
