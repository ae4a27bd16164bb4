"""B200 (sm_100a) implementation of ``com.microsoft.MatMulNBits`` for onnx-light.

``register_kernels()`` installs the operator into onnx-light's kernel dispatch table, the
way ``onnx_light_cpu.register_kernels()`` installs the CPU kernels; a model evaluated
afterwards runs MatMulNBits nodes on the GPU. ``MatMulNBitsSession`` runs a single node
through that same registered factory (host tensors in, host tensor out), and
``MatMulNBitsWeights`` is the device-pointer level used by benchmarks and sharded callers.
``qdq_to_matmulnbits`` / ``QdqMatMulSession`` take the standard-ONNX spelling of the same
projection (blocked ``DequantizeLinear`` of a constant weight, then ``MatMul``).
"""

from ._register import (
    RegisteredKernel,
    clear_used_kernel_names,
    register_kernels,
    registered_kernel_names,
    registered_kernels,
    set_kernel_usage_recording,
    used_kernel_names,
)
from .matmul_nbits import MatMulNBitsSession, MatMulNBitsWeights
from .qdq import QdqMatMulSession, qdq_to_matmulnbits

__version__ = "0.1.0"

__all__ = [
    "MatMulNBitsSession",
    "MatMulNBitsWeights",
    "QdqMatMulSession",
    "RegisteredKernel",
    "clear_used_kernel_names",
    "qdq_to_matmulnbits",
    "register_kernels",
    "registered_kernel_names",
    "registered_kernels",
    "set_kernel_usage_recording",
    "used_kernel_names",
]
