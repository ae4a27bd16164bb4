"""Isolated MatMulNBits kernel throughput on one B200.

CUDA counterpart of the reference's ``tools/compact_gemm_throughput.cc``: a fixed list of shapes,
device-resident operands, warm-up outside the samples, at least seven recorded samples, median
and inter-quartile range (never best-of), raw samples kept, environment metadata, optional JSON.
Weights rotate over enough copies to exceed the 126 MB L2 for memory-bound shapes.

    python -m onnx_light_cpu_b200.tools.nbits_throughput [--json out.json] [--samples 9]
"""

from __future__ import annotations

import argparse
import json
import platform
import statistics
import sys

L2_BYTES = 126 * 1024 * 1024

# name, M, K, N, bits, block_size, zero_points, bias, accuracy_level
SHAPES = (
    ("cfg1_single_node", 1, 4096, 4096, 4, 32, False, False, 0),
    ("cfg2_decode_m1", 1, 4096, 14336, 4, 128, True, True, 0),
    ("cfg2_decode_m4", 4, 4096, 14336, 4, 128, True, True, 0),
    ("cfg2_decode_m16", 16, 4096, 14336, 4, 128, True, True, 0),
    ("cfg3_prefill_m512", 512, 4096, 4096, 4, 64, True, False, 0),
    ("cfg3_prefill_m2048", 2048, 4096, 4096, 4, 64, True, False, 0),
    ("cfg3_prefill_m8192", 8192, 4096, 4096, 4, 64, True, False, 0),
    ("cfg4_gate_m16", 16, 4096, 14336, 4, 32, False, False, 0),
    ("cfg4_gate_m16_level4", 16, 4096, 14336, 4, 32, False, False, 4),
    ("cfg4_down_m16", 16, 14336, 4096, 4, 32, False, False, 0),
    ("cfg4_down_m16_level4", 16, 14336, 4096, 4, 32, False, False, 4),
    ("cfg2_decode_m1_level4", 1, 4096, 14336, 4, 128, True, True, 4),
    ("cfg2_decode_m16_level4", 16, 4096, 14336, 4, 128, True, True, 4),
    ("cfg5_shard8_m1", 1, 4096, 16032, 4, 32, True, False, 0),
    ("cfg5_shard8_m1_8bit", 1, 4096, 16032, 8, 32, True, False, 0),
    ("cfg5_shard8_m8", 8, 4096, 16032, 4, 32, True, False, 0),
    ("cfg5_shard8_m256", 256, 4096, 16032, 4, 32, True, False, 0),
    ("cfg5_shard8_m8_8bit", 8, 4096, 16032, 8, 32, True, False, 0),
    ("cfg5_shard8_m256_8bit", 256, 4096, 16032, 8, 32, True, False, 0),
    ("cfg5_shard8_m8_8bit_level4", 8, 4096, 16032, 8, 32, True, False, 4),
    # between decode and prefill: 17 <= M <= 256 on the decode geometry and the prefill geometry
    ("mid_cfg2_m32", 32, 4096, 14336, 4, 128, True, True, 0),
    ("mid_cfg2_m64", 64, 4096, 14336, 4, 128, True, True, 0),
    ("mid_cfg2_m128", 128, 4096, 14336, 4, 128, True, True, 0),
    ("mid_cfg2_m256", 256, 4096, 14336, 4, 128, True, True, 0),
    ("mid_cfg3_m64", 64, 4096, 4096, 4, 64, True, False, 0),
    ("mid_cfg3_m256", 256, 4096, 4096, 4, 64, True, False, 0),
    # shapes outside the staged kernels: 8-bit rows too long for whole-row stages, blocks of sixteen
    ("down8_m1", 1, 14336, 4096, 8, 128, True, False, 0),
    ("down8_m8", 8, 14336, 4096, 8, 128, True, False, 0),
    ("block16_m1", 1, 4096, 14336, 4, 16, True, False, 0),
    ("block16_m8", 8, 4096, 14336, 4, 16, True, False, 0),
)


def repeats_for(seconds_per_call: float, floor: int = 5, ceiling: int = 101, budget: float = 0.02) -> int:
    """Calls per sample so that one sample lasts about `budget` seconds, clamped like the
    reference tool clamps its repeat count."""
    if seconds_per_call <= 0:
        return ceiling
    return int(max(floor, min(ceiling, round(budget / seconds_per_call))))


def summarize(samples: list[float]) -> dict:
    ordered = sorted(samples)
    q = statistics.quantiles(ordered, n=4) if len(ordered) >= 4 else [ordered[0], statistics.median(ordered), ordered[-1]]
    return {"median": statistics.median(ordered), "iqr": q[2] - q[0], "min": ordered[0], "max": ordered[-1],
            "samples": list(samples)}


def copies_for(bytes_per_call: int) -> int:
    """Weight copies to rotate over so that consecutive calls cannot be served from L2."""
    return max(1, min(16, -(-2 * L2_BYTES // max(bytes_per_call, 1))))


def measure(shape, samples: int) -> dict:
    import torch

    import onnx_light_cpu_b200 as pkg
    from onnx_light_cpu_b200 import _capi

    name, m, k, n, bits, bs, zp, bias, level = shape
    nb = -(-k // bs)
    nbytes = _capi.algorithmic_bytes(m, n, k, bits, bs, zp, bias)
    copies = copies_for(nbytes)
    gen = torch.Generator(device="cuda")
    gen.manual_seed(0x404)
    weights = []
    for _ in range(copies):
        b = torch.randint(0, 256, (n, nb, bs * bits // 8), dtype=torch.uint8, device="cuda", generator=gen)
        sc = torch.randn(n * nb, device="cuda", generator=gen).abs() * 0.02
        z = torch.randint(0, 256, (n, (nb * bits + 7) // 8), dtype=torch.uint8, device="cuda", generator=gen) if zp else None
        bi = torch.randn(n, device="cuda", generator=gen) * 0.1 if bias else None
        weights.append(pkg.MatMulNBitsWeights(b, sc, z, bi, K=k, N=n, bits=bits, block_size=bs))
    a = torch.randn(m, k, device="cuda", generator=gen)
    y = torch.empty(m, n, device="cuda")

    def one_pass():
        for w in weights:
            w.matmul_device(a, y, accuracy_level=level)

    for _ in range(3):
        one_pass()
    torch.cuda.synchronize()
    kernel = _capi.last_kernel()
    status = max(w.poll_status() for w in weights)
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    begin.record()
    one_pass()
    end.record()
    torch.cuda.synchronize()
    reps = repeats_for(begin.elapsed_time(end) / 1e3)
    times = []
    for _ in range(max(samples, 7)):
        begin.record()
        for _ in range(reps):
            one_pass()
        end.record()
        torch.cuda.synchronize()
        times.append(begin.elapsed_time(end) / 1e3 / (reps * copies))
    stats = summarize(times)
    flops = 2.0 * m * n * k
    out = {"shape": name, "m": m, "k": k, "n": n, "bits": bits, "block_size": bs, "accuracy_level": level,
           "kernel": kernel, "device_status": status, "weight_copies": copies, "calls_per_sample": reps * copies,
           "seconds": stats, "gbs_median": nbytes / stats["median"] / 1e9,
           "tflops_median": flops / stats["median"] / 1e12, "algorithmic_bytes": nbytes}
    for w in weights:
        w.close()
    return out


def metadata() -> dict:
    import torch

    props = torch.cuda.get_device_properties(0)
    return {"platform": platform.platform(), "python": sys.version.split()[0], "torch": torch.__version__,
            "gpu": props.name, "sm_count": props.multi_processor_count, "cuda": torch.version.cuda,
            "weights": "constant, device resident (uploaded once)", "timing": "CUDA events, median of samples"}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--json", default=None)
    parser.add_argument("--samples", type=int, default=9)
    parser.add_argument("--only", default=None, help="substring filter on the shape name")
    args = parser.parse_args(argv)
    import torch

    if not torch.cuda.is_available():
        print("nbits_throughput needs a CUDA device", file=sys.stderr)
        return 1
    rows = [measure(shape, args.samples) for shape in SHAPES if args.only is None or args.only in shape[0]]
    print(f"{'shape':26s} {'kernel':34s} {'us/call':>9s} {'iqr us':>8s} {'GB/s':>8s} {'TFLOP/s':>8s}")
    for r in rows:
        print(f"{r['shape']:26s} {r['kernel'][:34]:34s} {r['seconds']['median'] * 1e6:9.2f} "
              f"{r['seconds']['iqr'] * 1e6:8.2f} {r['gbs_median']:8.1f} {r['tflops_median']:8.2f}")
    if args.json:
        with open(args.json, "w") as handle:
            json.dump({"metadata": metadata(), "results": rows}, handle, indent=1)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
