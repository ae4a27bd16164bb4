"""Seeded synthetic MatMulNBits inputs with the shapes and value distributions of the five
benchmark configurations. No dataset or model weights are involved: every value is drawn
from ``numpy.random.default_rng(seed)`` in the fixed order A, B, scales, zero_points, bias.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np


@dataclass
class Case:
    name: str
    m: int
    k: int
    n: int
    bits: int
    block_size: int
    a: np.ndarray
    b: np.ndarray
    scales: np.ndarray
    zero_points: np.ndarray | None
    bias: np.ndarray | None
    accuracy_level: int = 0
    meta: dict = field(default_factory=dict)

    @property
    def n_blocks(self) -> int:
        return -(-self.k // self.block_size)


def make_case(name, m, k, n, bits, block_size, *, seed, a_dist="normal", scale_sigma=0.02,
              scale_floor=0.0, zero_points=True, bias=False, fp16_a=False, accuracy_level=0) -> Case:
    rng = np.random.default_rng(seed)
    n_blocks = -(-k // block_size)
    blob = block_size * bits // 8
    if a_dist == "uniform":
        a = rng.uniform(-1.0, 1.0, size=(m, k)).astype(np.float32)
    else:
        a = rng.standard_normal(size=(m, k), dtype=np.float32)
    if fp16_a:
        a = a.astype(np.float16).astype(np.float32)
    b = rng.integers(0, 256, size=(n, n_blocks, blob), dtype=np.uint8)
    scales = (np.abs(rng.standard_normal(size=(n * n_blocks,), dtype=np.float32)) * np.float32(scale_sigma)
              + np.float32(scale_floor)).astype(np.float32)
    zp = None
    if zero_points:
        zp = rng.integers(0, 256, size=(n, (n_blocks * bits + 7) // 8), dtype=np.uint8)
    bias_arr = None
    if bias:
        bias_arr = (rng.standard_normal(size=(n,), dtype=np.float32) * np.float32(0.1)).astype(np.float32)
    return Case(name, m, k, n, bits, block_size, a, b, scales, zp, bias_arr, accuracy_level,
                {"seed": seed})


# The five configurations. Seeds: cfg1 is fixed to 0 by its definition; the others are
# 1000 + 100*config + variant.
def config1() -> Case:
    return make_case("cfg1_single_node", 1, 4096, 4096, 4, 32, seed=0, a_dist="uniform",
                     scale_sigma=0.02, scale_floor=1e-4, zero_points=False, bias=False)


def config2(m: int = 1, n: int = 14336) -> Case:
    return make_case(f"cfg2_decode_m{m}", m, 4096, n, 4, 128, seed=1200 + m, scale_sigma=0.01,
                     zero_points=True, bias=True, fp16_a=True)


def config3(m: int = 2048, n: int = 4096) -> Case:
    return make_case(f"cfg3_prefill_m{m}", m, 4096, n, 4, 64, seed=1300 + (m % 97), scale_sigma=0.02,
                     zero_points=True, bias=False)


LLAMA_LAYER = (("q", 4096, 4096), ("k", 4096, 1024), ("v", 4096, 1024), ("o", 4096, 4096),
               ("gate", 4096, 14336), ("up", 4096, 14336), ("down", 14336, 4096))


def config4(accuracy_level: int = 0, m: int = 16) -> list[Case]:
    return [make_case(f"cfg4_{name}", m, k, n, 4, 32, seed=1400 + i, scale_sigma=0.02, zero_points=False,
                      bias=False, accuracy_level=accuracy_level)
            for i, (name, k, n) in enumerate(LLAMA_LAYER)]


def config5(m: int = 1, bits: int = 4, n: int = 128256) -> Case:
    return make_case(f"cfg5_lmhead_m{m}_b{bits}", m, 4096, n, bits, 32, seed=1500 + m + bits,
                     scale_sigma=0.02, zero_points=True, bias=False)


def shard_columns(case: Case, world_size: int, rank: int) -> Case:
    """Column shard ``rank`` of ``world_size``: contiguous N range, A replicated. When N does not
    divide, the first ``N % world_size`` shards are one column wider."""
    per, extra = divmod(case.n, world_size)
    lo = per * rank + min(rank, extra)
    hi = lo + per + (1 if rank < extra else 0)
    nb = case.n_blocks
    return Case(f"{case.name}_shard{rank}of{world_size}", case.m, case.k, hi - lo, case.bits, case.block_size,
                case.a, case.b[lo:hi], case.scales.reshape(case.n, nb)[lo:hi].reshape(-1),
                None if case.zero_points is None else case.zero_points[lo:hi],
                None if case.bias is None else case.bias[lo:hi], case.accuracy_level,
                dict(case.meta, col_offset=lo))


def algorithmic_bytes(m: int, n: int, k: int, bits: int, block_size: int, has_zero_points: bool,
                      has_bias: bool) -> int:
    """Bytes the operator must read and write once per call (packed weights, scales, zero points,
    bias, A, Y): the figure every roofline number is computed from. Same formula as the C ABI's
    ``mnb_algorithmic_bytes``; restated here so that the CPU legs need not load the CUDA library."""
    n_blocks = -(-k // block_size)
    total = n * n_blocks * (block_size * bits // 8) + 4 * n * n_blocks
    if has_zero_points:
        total += n * ((n_blocks * bits + 7) // 8)
    if has_bias:
        total += 4 * n
    return total + 4 * m * k + 4 * m * n
