"""End-to-end parity + speed of single-node MatMulNBits models: registered GPU operator versus
the CPU restatement, alternating.

Counterpart of the reference's ``tools/benchmark_integer_gemm_parity.py`` (which alternates the
registered ``MatMulInteger`` kernel with ONNX Runtime): seeded inputs per case, a parity check
before timing, warm-up outside the samples, garbage collection off while timing, the order of
the two candidates rotating every iteration, median / IQR / raw samples, a speed gate
(median >= 1.0, minimum >= 0.9 over the corpus). The CPU side is the operator's CPU restatement
(the reference ships no MatMulNBits kernel); it is loaded from ``oracle/`` and is the checker,
not a product path.

    python -m onnx_light_cpu_b200.tools.benchmark_nbits_parity [--json out.json] [--threads N]
"""

from __future__ import annotations

import argparse
import gc
import json
import statistics
import sys
import time
from pathlib import Path

# name, M, K, N, bits, block_size, zero_points, bias, accuracy_level, tolerance
CORPUS = (
    ("decode_m1_b128", 1, 4096, 14336, 4, 128, True, True, 0, 1e-5),
    ("decode_m1_b32", 1, 4096, 4096, 4, 32, False, False, 0, 1e-5),
    ("decode_m4_b128", 4, 4096, 4096, 4, 128, True, False, 0, 1e-5),
    ("decode_m1_8bit", 1, 4096, 4096, 8, 32, True, False, 0, 1e-5),
    ("prefill_m256_b64", 256, 4096, 1024, 4, 64, True, False, 0, 2e-2),
    ("level4_m16_b32", 16, 4096, 4096, 4, 32, False, False, 4, 2e-2),
)


def speed_gate(speedups: list[float], median_floor: float = 1.0, min_floor: float = 0.9) -> dict:
    """Pass/fail of the corpus: median speed-up and slowest case against their floors."""
    if not speedups:
        return {"passed": False, "median": None, "min": None}
    med, low = statistics.median(speedups), min(speedups)
    return {"passed": med >= median_floor and low >= min_floor, "median": med, "min": low,
            "median_floor": median_floor, "min_floor": min_floor}


def measure_alternating(first, second, iterations: int, warmup: int = 2) -> tuple[list[float], list[float]]:
    """Times two callables alternately; the one that goes first changes every iteration."""
    for _ in range(warmup):
        first()
        second()
    a_times, b_times = [], []
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        for i in range(iterations):
            order = ((first, a_times), (second, b_times)) if i % 2 == 0 else ((second, b_times), (first, a_times))
            for fn, sink in order:
                t0 = time.perf_counter_ns()
                fn()
                sink.append((time.perf_counter_ns() - t0) / 1e9)
    finally:
        if was_enabled:
            gc.enable()
    return a_times, b_times


def stats(samples: list[float]) -> dict:
    ordered = sorted(samples)
    q = statistics.quantiles(ordered, n=4) if len(ordered) >= 4 else [ordered[0], ordered[len(ordered) // 2], ordered[-1]]
    return {"median": statistics.median(ordered), "iqr": q[2] - q[0], "samples": list(samples)}


def run(threads: int | None, iterations: int) -> dict:
    import numpy as np

    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    import onnx_light_cpu_b200 as pkg
    from onnx_light_cpu_b200.tools import synthetic as syn
    from oracle import nbits_oracle as o

    pkg.register_kernels()
    pkg.set_kernel_usage_recording(False)  # keep the log's mutex out of the timings
    threads = threads or o.hardware_threads()
    rows, speedups = [], []
    for index, (name, m, k, n, bits, bs, zp, bias, level, tol) in enumerate(CORPUS):
        case = syn.make_case(name, m, k, n, bits, bs, seed=index, zero_points=zp, bias=bias)
        session = pkg.MatMulNBitsSession(case.b, case.scales, case.zero_points, case.bias, K=k, N=n, bits=bits,
                                         block_size=bs, accuracy_level=level)
        cpu = o.matmul_int8 if level == 4 else o.matmul_f32_fast
        args = (case.a, case.b, case.scales, case.zero_points, case.bias, n, k, bits, bs)
        got = session.run(case.a)
        ref = o.matmul_f64(*args)
        err = float(np.abs(got - ref).max() / np.abs(ref).max())
        parity_ok = err <= (tol if level == 0 else 2e-2)
        gpu_t, cpu_t = measure_alternating(lambda: session.run(case.a), lambda: cpu(*args, threads=threads), iterations)
        g, c = stats(gpu_t), stats(cpu_t)
        speedup = c["median"] / g["median"]
        speedups.append(speedup)
        rows.append({"case": name, "kernel": session.last_device_kernel, "rel_err": err, "parity_ok": parity_ok,
                     "gpu_seconds": g, "cpu_seconds": c, "speedup": speedup})
        session.close()
    return {"threads": threads, "cpu_side": "CPU restatement of MatMulNBits (not a reference kernel)",
            "layer": "end to end through the registered operator: host tensors in and out, constant weights",
            "results": rows, "gate": speed_gate(speedups), "parity": all(r["parity_ok"] for r in rows)}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--json", default=None)
    parser.add_argument("--threads", type=int, default=None)
    parser.add_argument("--iterations", type=int, default=15)
    args = parser.parse_args(argv)
    report = run(args.threads, args.iterations)
    for r in report["results"]:
        print(f"{r['case']:20s} {r['kernel'][:30]:30s} err {r['rel_err']:.2e}  gpu {r['gpu_seconds']['median'] * 1e6:9.1f} us"
              f"  cpu {r['cpu_seconds']['median'] * 1e6:10.1f} us  x{r['speedup']:.1f}")
    print("gate:", report["gate"], "parity:", report["parity"])
    if args.json:
        with open(args.json, "w") as handle:
            json.dump(report, handle, indent=1)
    return 0 if report["parity"] and report["gate"]["passed"] else 1


if __name__ == "__main__":
    raise SystemExit(main())
