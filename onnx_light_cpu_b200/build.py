"""Builds the native libraries of this package in-tree.

``libmatmulnbits_b200.so``  hand-written sm_100a CUDA kernels + the C ABI (nvcc)
``libonnx_light_cuda_kernels.so``  C++ operator class, registration layer and the ctypes bridge (g++)

``python -m onnx_light_cpu_b200.build`` or :func:`build_all`. nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import os
import subprocess
import sys
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
REPO_ROOT = PACKAGE_DIR.parent
CUDA_LIB = PACKAGE_DIR / "libmatmulnbits_b200.so"
HOST_LIB = PACKAGE_DIR / "libonnx_light_cuda_kernels.so"

CUDA_SOURCES = [
    "csrc/c_api.cu",
    "csrc/nbits_gemv.cu",
    "csrc/nbits_gemv_mma.cu",
    "csrc/nbits_gemv_mma_multi.cu",
    "csrc/nbits_gemv_imma.cu",
    "csrc/nbits_gemv_u8_mma.cu",
    "csrc/nbits_decode_direct.cu",
    "csrc/nbits_decode_resident.cu",
    "csrc/nbits_int8.cu",
    "csrc/nbits_int8_mma.cu",
    "csrc/nbits_gemm_tcgen05.cu",
]
CUDA_HEADERS = ["csrc/nbits_common.cuh", "csrc/nbits_digits.cuh", "csrc/nbits_ptx.cuh", "csrc/nbits_tma.cuh", "csrc/nbits_mma_common.cuh",
                "../include/matmulnbits_b200.h"]
HOST_SOURCES = [
    "kernels/kernel_registration.cc",
    "kernels/kernel_usage.cc",
    "kernels/register_kernels.cc",
    "kernels/math/matmul_nbits_kernel.cc",
    "kernels/parallel/peer_gather.cc",
    "onnx_py/cudaregister_capi.cc",
]
HOST_HEADERS = [
    "kernels/kernel_registration.h",
    "kernels/kernel_usage.h",
    "kernels/register_kernels.h",
    "kernels/math/matmul_nbits_kernel.h",
    "kernels/parallel/peer_gather.h",
    "shim/onnx_core/onnx_light_shim.h",
    "../include/matmulnbits_b200.h",
]

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "-Xcompiler",
    "-fPIC",
    "-shared",
]


def _nvcc() -> str:
    for candidate in (os.environ.get("NVCC"), "/usr/local/cuda/bin/nvcc", "nvcc"):
        if candidate and (os.path.sep not in candidate or os.path.exists(candidate)):
            return candidate
    return "nvcc"


def _stale(target: Path, inputs: list[str]) -> bool:
    if not target.exists():
        return True
    stamp = target.stat().st_mtime
    return any((PACKAGE_DIR / name).stat().st_mtime > stamp for name in inputs)


def _run(command: list[str]) -> None:
    result = subprocess.run(command, cwd=PACKAGE_DIR, capture_output=True, text=True)
    if result.returncode != 0:
        raise RuntimeError("build failed: " + " ".join(command) + "\n" + result.stdout + result.stderr)
    if "-v" in command and result.stderr:
        print(result.stderr, file=sys.stderr)


def build_cuda(force: bool = False, verbose_ptxas: bool = False) -> Path:
    """One object file per source (compiled in parallel, rebuilt only when the source or a header
    is newer), then one link. Objects live in ``build/`` beside the package sources."""
    if not (force or verbose_ptxas or _stale(CUDA_LIB, CUDA_SOURCES + CUDA_HEADERS)):
        return CUDA_LIB
    headers_stamp = max((PACKAGE_DIR / name).stat().st_mtime for name in CUDA_HEADERS)
    objects_dir = PACKAGE_DIR / "build"
    objects_dir.mkdir(exist_ok=True)
    compile_flags = [flag for flag in NVCC_FLAGS if flag != "-shared"]
    if verbose_ptxas:
        compile_flags += ["-Xptxas", "-v"]
    jobs, objects = [], []
    for source in CUDA_SOURCES:
        obj = objects_dir / (Path(source).stem + ".o")
        objects.append(str(obj))
        stamp = max((PACKAGE_DIR / source).stat().st_mtime, headers_stamp)
        if force or verbose_ptxas or not obj.exists() or obj.stat().st_mtime < stamp:
            jobs.append([_nvcc(), *compile_flags, "-c", "-o", str(obj), source])
    if jobs:
        from concurrent.futures import ThreadPoolExecutor

        with ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as pool:
            list(pool.map(_run, jobs))
    if jobs or not CUDA_LIB.exists():
        _run([_nvcc(), "-shared", "-o", str(CUDA_LIB), *objects])
    return CUDA_LIB


def build_host(force: bool = False, onnx_light_include: str | None = None) -> Path:
    """Compiles the operator class against onnx-light's headers when ``onnx_light_include``
    (or the environment variable ONNX_LIGHT_INCLUDE_DIR) names them, else against the
    stand-in headers under ``shim/``."""
    include = onnx_light_include or os.environ.get("ONNX_LIGHT_INCLUDE_DIR")
    if force or _stale(HOST_LIB, HOST_SOURCES + HOST_HEADERS) or _stale(HOST_LIB, ["libmatmulnbits_b200.so"]):
        command = [os.environ.get("CXX", "g++"), "-std=c++20", "-O2", "-fPIC", "-Wall", "-Wextra", "-shared",
                   "-I", str(REPO_ROOT)]
        if include:
            command += ["-I", include]
        command += ["-I", str(PACKAGE_DIR / "shim"), "-o", str(HOST_LIB), *HOST_SOURCES,
                    "-L", str(PACKAGE_DIR), "-lmatmulnbits_b200", "-Wl,-rpath,$ORIGIN"]
        _run(command)
    return HOST_LIB


def build_all(force: bool = False) -> None:
    build_cuda(force)
    build_host(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print(CUDA_LIB)
    print(HOST_LIB)
