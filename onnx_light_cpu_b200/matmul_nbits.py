"""Python-level objects over the native libraries.

* :class:`MatMulNBitsSession` - one MatMulNBits node evaluated through the registered C++
  kernel factory, numpy arrays in and out (what a user of the evaluator sees).
* :class:`MatMulNBitsWeights` - the C ABI at device-pointer level; takes ``torch`` CUDA
  tensors only as owners of device memory and streams.
"""

from __future__ import annotations

import ctypes

import numpy as np

from . import _capi
from . import _register


def _ptr(array: np.ndarray | None) -> ctypes.c_void_p | None:
    return None if array is None else ctypes.c_void_p(array.ctypes.data)


class MatMulNBitsSession:
    """Single-node model ``Y = MatMulNBits(A, B, scales[, zero_points][, bias])`` whose kernel
    is built by the factory that ``register_kernels()`` installed. Constant operands are
    copied into the session (initializer lifetime); every :meth:`run` uploads ``A``, runs on
    the GPU and returns ``Y`` as a new numpy array."""

    def __init__(self, b, scales, zero_points=None, bias=None, *, K, N, bits=4, block_size=32,
                 accuracy_level=0, _with_g_idx=False):
        lib = _register._host_lib()
        self._lib = lib
        self.n = int(N)
        self.k = int(K)
        b = np.ascontiguousarray(b, dtype=np.uint8)
        scales = np.ascontiguousarray(scales, dtype=np.float32)
        zp = None if zero_points is None else np.ascontiguousarray(zero_points, dtype=np.uint8)
        bias_arr = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
        self._handle = lib.olc_session_create(
            _ptr(b), b.size, _ptr(scales), scales.size, _ptr(zp), 0 if zp is None else zp.size,
            _ptr(bias_arr), 0 if bias_arr is None else bias_arr.size, int(K), int(N), int(bits),
            int(block_size), int(accuracy_level), 1 if _with_g_idx else 0)
        if not self._handle:
            message = lib.olc_last_error().decode()
            raise RuntimeError(message)

    def run(self, a: np.ndarray) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        shape = (ctypes.c_int64 * a.ndim)(*a.shape)
        lead = a.shape[:-1]
        y = np.empty(lead + (self.n,), dtype=np.float32)
        code = self._lib.olc_session_run(self._handle, _ptr(a), shape, a.ndim, _ptr(y), y.size)
        if code != 0:
            _register._raise_last(code)
        return y

    def overwrite_b(self, b) -> None:
        """Rewrites the session's initializer ``B`` in place (same buffer): the next :meth:`run`
        must notice and upload the new weights."""
        b = np.ascontiguousarray(b, dtype=np.uint8)
        code = self._lib.olc_session_overwrite_b(self._handle, _ptr(b), b.size)
        if code != 0:
            _register._raise_last(code)

    @property
    def last_device_kernel(self) -> str:
        return self._lib.olc_session_last_device_kernel(self._handle).decode()

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.olc_session_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def _check_device_tensor(what, tensor, dtype_name, device, min_elements=0):
    """The C ABI takes raw addresses: a tensor of the wrong dtype, on the host, on another GPU, not
    contiguous or too small would become an out-of-bounds device access, so it is refused here."""
    if not getattr(tensor, "is_cuda", False):
        raise ValueError(f"{what} must be a CUDA tensor")
    if str(tensor.dtype) != "torch." + dtype_name:
        raise ValueError(f"{what} must have dtype {dtype_name}, got {tensor.dtype}")
    if not tensor.is_contiguous():
        raise ValueError(f"{what} must be contiguous")
    if (tensor.device.index or 0) != device:
        raise ValueError(f"{what} is on GPU {tensor.device.index}, the weights are on GPU {device}")
    if tensor.numel() < min_elements:
        raise ValueError(f"{what} holds {tensor.numel()} elements, {min_elements} are needed")


MAX_GROUPED_NODES = 3


def matmul_device_group(nodes, a, ys, accuracy_level=0, stream=None) -> None:
    """Sibling nodes that take the same activations (q / k / v, gate / up) in one call:
    ``ys[i] = nodes[i](a)``, each ``ys[i]`` a dense fp32 CUDA tensor [m, N_i]. One to three
    :class:`MatMulNBitsWeights` with the same K on the same GPU. Asynchronous on ``stream``."""
    import ctypes

    import torch

    nodes = list(nodes)
    ys = list(ys)
    if not 1 <= len(nodes) <= MAX_GROUPED_NODES or len(ys) != len(nodes):
        raise ValueError(f"a group takes 1 to {MAX_GROUPED_NODES} nodes and as many outputs")
    first = nodes[0]
    m = first._rows_of(a)
    for node, y in zip(nodes, ys):
        if node.k != first.k or node.device != first.device:
            raise ValueError("the nodes of a group take the same activations: same K, same GPU")
        _check_device_tensor("y", y, "float32", node.device, m * node.n)
    raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
    handles = (ctypes.c_void_p * len(nodes))(*[node._handle for node in nodes])
    outputs = (ctypes.c_void_p * len(nodes))(*[y.data_ptr() for y in ys])
    _capi.check(first._lib.mnb_matmul_device_group(handles, len(nodes), a.data_ptr(), m, accuracy_level, outputs, raw))


class MatMulNBitsWeights:
    """Device-resident weights of one node plus the device-pointer entry points.

    ``b``, ``scales``, ``zero_points``, ``bias`` are either numpy arrays (uploaded once) or
    torch CUDA tensors (wrapped without a copy and kept alive by this object)."""

    def __init__(self, b, scales, zero_points=None, bias=None, *, K, N, bits=4, block_size=32, device=0):
        self._lib = _capi.load()
        self.k, self.n, self.bits, self.block_size = int(K), int(N), int(bits), int(block_size)
        self.has_zero_points = zero_points is not None
        self.has_bias = bias is not None
        handle = ctypes.c_void_p()
        if isinstance(b, np.ndarray):
            b = np.ascontiguousarray(b, dtype=np.uint8)
            scales = np.ascontiguousarray(scales, dtype=np.float32)
            zp = None if zero_points is None else np.ascontiguousarray(zero_points, dtype=np.uint8)
            bias_arr = None if bias is None else np.ascontiguousarray(bias, dtype=np.float32)
            _capi.check(self._lib.mnb_weights_create(
                device, _ptr(b), _ptr(scales), _ptr(zp), _ptr(bias_arr), self.n, self.k, self.bits,
                self.block_size, ctypes.byref(handle)))
            self._keep = ()
        else:
            self._keep = (b, scales, zero_points, bias)
            device = b.device.index or 0
            _capi.check(self._lib.mnb_weights_wrap_device(
                device, b.data_ptr(), scales.data_ptr(),
                None if zero_points is None else zero_points.data_ptr(),
                None if bias is None else bias.data_ptr(), self.n, self.k, self.bits, self.block_size,
                ctypes.byref(handle)))
        self._handle = handle
        self.device = device

    def algorithmic_bytes(self, m: int) -> int:
        return _capi.algorithmic_bytes(m, self.n, self.k, self.bits, self.block_size,
                                       self.has_zero_points, self.has_bias)

    def matmul_host(self, a: np.ndarray, accuracy_level=0, path=_capi.PATH_AUTO, out=None) -> np.ndarray:
        a = np.ascontiguousarray(a, dtype=np.float32)
        m = a.size // self.k
        y = out if out is not None else np.empty((m, self.n), dtype=np.float32)
        _capi.check(self._lib.mnb_matmul_host(self._handle, _ptr(a), m, accuracy_level, path, _ptr(y)))
        return y

    def matmul_host_ptr(self, a_ptr: int, m: int, y_ptr: int, accuracy_level=0, path=_capi.PATH_AUTO) -> None:
        """Host-buffer call on raw addresses (e.g. pinned torch tensors)."""
        _capi.check(self._lib.mnb_matmul_host(self._handle, a_ptr, m, accuracy_level, path, y_ptr))

    def matmul_device(self, a, y, accuracy_level=0, path=_capi.PATH_AUTO, stream=None,
                      ld_y=None, col_offset=0) -> None:
        """``a`` [m, K] and ``y`` torch CUDA fp32 tensors; asynchronous on ``stream`` (a
        ``torch.cuda.Stream``; default: the current stream)."""
        import torch

        m = self._rows_of(a)
        ld = self.n if ld_y is None else int(ld_y)
        if col_offset < 0 or col_offset + self.n > ld:
            raise ValueError("the output window [col_offset, col_offset + N) does not fit a row of ld_y elements")
        _check_device_tensor("y", y, "float32", self.device, (m - 1) * ld + col_offset + self.n if m > 0 else 0)
        raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
        _capi.check(self._lib.mnb_matmul_device_strided(
            self._handle, a.data_ptr(), m, accuracy_level, path, y.data_ptr(),
            self.n if ld_y is None else ld_y, col_offset, raw))

    def matmul_int8_static(self, a, y, stream=None) -> None:
        """accuracy_level-4 product through the entry point that allocates nothing (its
        activation scratch is a fixed array inside the library; limits in the C header).
        ``a`` [m, K] and ``y`` [m, N] are torch CUDA fp32 tensors."""
        import torch

        m = self._rows_of(a)
        _check_device_tensor("y", y, "float32", self.device, m * self.n)
        raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
        _capi.check(self._lib.mnb_matmul_int8_static(self._handle, a.data_ptr(), m, y.data_ptr(), raw))

    def _rows_of(self, a) -> int:
        _check_device_tensor("a", a, "float32", self.device)
        if a.numel() % self.k != 0:
            raise ValueError(f"a holds {a.numel()} elements, not a multiple of K = {self.k}")
        return a.numel() // self.k

    def poll_status(self) -> int:
        status = ctypes.c_int(0)
        _capi.check(self._lib.mnb_weights_poll_status(self._handle, ctypes.byref(status)))
        return status.value

    def dequant_int(self, out, stream=None) -> None:
        import torch

        _check_device_tensor("out", out, "int32", self.device, self.n * self.k)
        raw = (stream or torch.cuda.current_stream(out.device)).cuda_stream
        _capi.check(self._lib.mnb_dequant_int_device(self._handle, out.data_ptr(), raw))

    def int8_block_dots(self, aq, dots, stream=None) -> None:
        import torch

        _check_device_tensor("aq", aq, "int8", self.device)
        if aq.numel() % self.k != 0:
            raise ValueError(f"aq holds {aq.numel()} elements, not a multiple of K = {self.k}")
        raw = (stream or torch.cuda.current_stream(aq.device)).cuda_stream
        m = aq.numel() // self.k
        n_blocks = -(-self.k // self.block_size)
        _check_device_tensor("dots", dots, "int32", self.device, m * self.n * n_blocks)
        _capi.check(self._lib.mnb_int8_block_dots_device(self._handle, aq.data_ptr(), m, dots.data_ptr(), raw))

    def int8_mma_block_dots(self, a, y, dots, stream=None) -> None:
        """accuracy_level-4 product through the instrumented form of the integer-MMA kernel: ``y``
        [m, N] fp32 as usual, ``dots`` [m, N, n_blocks] int32 = the kernel's exact block sums."""
        import torch

        m = self._rows_of(a)
        n_blocks = -(-self.k // self.block_size)
        _check_device_tensor("y", y, "float32", self.device, m * self.n)
        _check_device_tensor("dots", dots, "int32", self.device, m * self.n * n_blocks)
        raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
        _capi.check(self._lib.mnb_int8_mma_block_dots_device(self._handle, a.data_ptr(), m, y.data_ptr(),
                                                             dots.data_ptr(), raw))

    def close(self) -> None:
        if getattr(self, "_handle", None):
            self._lib.mnb_weights_destroy(self._handle)
            self._handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def quantize_a(a, aq, a_scales, block_size: int, stream=None) -> None:
    """accuracy_level-4 activation quantization on device tensors (parity hook)."""
    import torch

    lib = _capi.load()
    k = a.shape[-1]
    m = a.numel() // k
    raw = (stream or torch.cuda.current_stream(a.device)).cuda_stream
    _capi.check(lib.mnb_quantize_a_device(a.data_ptr(), m, k, block_size, aq.data_ptr(), a_scales.data_ptr(), raw))
