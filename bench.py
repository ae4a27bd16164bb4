#!/usr/bin/env python
"""Benchmark of the B200 MatMulNBits path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout (rank 0). Headline metric: effective HBM GB/s of the 4-bit decode
GEMV at M=1 (algorithmic bytes / device time), with the M=2048 and M=8192 prefill TFLOP/s, the
decode sweep, the roofline fractions and a timed CPU baseline in the same line.

N = 1   workload = the decode configuration the metric is quoted on: M=1, K=4096, N=14336,
        bits=4, block_size=128, zero points and bias. A step is one pass over R=8 distinct
        weight copies (252 MB, twice the 126 MB L2, so every launch streams from HBM),
        captured as one CUDA graph.
N > 1   workload = the large-N output projection (K=4096, N=128256, bits=4, block 32, M=1),
        weight columns sharded across ranks, every rank's columns stored into every rank's gathered
        result by the kernel itself (peer-mapped memory; `--gather nccl`: an all-gather behind the
        kernel); strong scaling (the total problem is fixed). A step is one pass over R=2 weight
        copies. Before timing, one gathered step is compared with the ranks' own products. The line
        carries `scaling_base`: the same node unsharded on one GPU, timed by rank 0 in the same run.

`value` times device-resident inputs; `e2e` goes through the host-buffer C ABI call (pinned
host A in, pinned host Y out, copies inside the timed region). `--impl reference` times the CPU
restatement of the operator (the reference ships no MatMulNBits kernel) on the host cores.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

DECODE = dict(k=4096, n=14336, bits=4, block_size=128)
PREFILL = dict(m=2048, k=4096, n=4096, bits=4, block_size=64)
LMHEAD = dict(k=4096, n=128256, bits=4, block_size=32)
L2_BYTES = 126 * 1024 * 1024

# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the decode kernels on the
# decode workload, each from one ncu capture of that kernel on this workload. A constant, not a
# measurement of the run: reported as `traffic`, with `traffic_source` saying so.
NCU_DECODE_TRAFFIC_BYTES = {
    "nbits_decode_resident_kernel": 31_793_920,
    "nbits_decode_direct_kernel": 31_538_688,
    "nbits_gemv_imma_kernel": 31_796_480,
    "nbits_gemv_mma_kernel": 32_258_304,
}
WORKLOAD_DECODE = "cfg2 decode M=1 K=4096 N=14336 bits=4 block=128 zp+bias"
WORKLOAD_LMHEAD = "cfg5 lm-head M=1 K=4096 N=128256 bits=4 block=32 zp, column shards gathered"


def workload_config(multi: bool, copies: int, bytes_per_launch: int) -> dict:
    """The `config` object, identical in both arms of a run."""
    return {"workload": WORKLOAD_LMHEAD if multi else WORKLOAD_DECODE, "weight_copies": copies,
            "bytes_per_launch": int(bytes_per_launch),
            "l2_defeat": f"{copies} weight copies = {copies * bytes_per_launch / 1e6:.0f} MB > 126 MB L2"}


def measured_peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        data = json.loads(path.read_text())
        return ({"hbm_gbs": float(data["hbm_gbs"]), "bf16_tflops": float(data["bf16_tflops"]),
                 "bf16_tflops_sustained": float(data.get("bf16_tflops_sustained", data["bf16_tflops"]))},
                "measured")
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples: list[list[str]] = []
        self._stop = threading.Event()
        self._thread = threading.Thread(target=self._loop, daemon=True)

    def _loop(self):
        while not self._stop.is_set():
            try:
                out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                      "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5)
                if out.returncode == 0 and out.stdout.strip():
                    self.samples.append([v.strip() for v in out.stdout.strip().split(",")])
            except Exception:
                pass
            self._stop.wait(0.1)

    def __enter__(self):
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def hold(self, step, torch, seconds: float = 1.0) -> None:
        """Keeps replaying `step` for about `seconds` with the sampler running: the timed region of
        the decode workload lasts tens of milliseconds, less than one nvidia-smi query, so the
        clocks are also sampled over a longer window of the very same launches."""
        self.window_seconds = seconds
        deadline = time.perf_counter() + seconds
        while time.perf_counter() < deadline:
            for _ in range(20):
                step()
            torch.cuda.synchronize()

    def summary(self) -> dict:
        mhz = [float(s[0]) for s in self.samples if s and s[0].replace(".", "").isdigit()]
        max_mhz = [float(s[1]) for s in self.samples if len(s) > 1 and s[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [name for i, name in enumerate(names)
                   if any(len(s) > 2 + i and s[2 + i].lower().startswith("active") for s in self.samples)]
        out = {"sm_mhz": statistics.median(mhz) if mhz else None, "sm_max_mhz": max(max_mhz) if max_mhz else None,
               "reasons": reasons, "samples": len(self.samples)}
        if getattr(self, "window_seconds", None):
            out["window"] = (f"timed region, then {self.window_seconds:.1f} s of the same step "
                             "(one nvidia-smi query takes longer than the timed region)")
        return out


def cpu_threading(o) -> str:
    """Turns on the reference's own threading for the CPU legs where oracle/_ref carries it."""
    if o.use_reference_execute_ranges(True):
        return "reference ExecuteRanges + persistent std::thread executor (ExecutionExecutorScope)"
    return "checker's own persistent worker pool (oracle/_ref absent)"


def cpu_port_baseline(seconds: float = 3.0) -> dict:
    """Times the CPU restatement (oracle port) on this host: M=1 decode workload, all threads."""
    from onnx_light_cpu_b200.tools import synthetic as syn
    from oracle import nbits_oracle as o

    case = syn.config2(1)
    threads = o.hardware_threads()
    threading_kind = cpu_threading(o)
    args = (case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, case.bits, case.block_size)
    for _ in range(3):   # the first call starts the worker threads
        o.matmul_f32_fast(*args, threads=threads)
    calls, start = 0, time.perf_counter()
    samples = []
    while time.perf_counter() - start < seconds or calls < 7:
        t0 = time.perf_counter()
        o.matmul_f32_fast(*args, threads=threads)
        samples.append(time.perf_counter() - t0)
        calls += 1
    nbytes = syn.algorithmic_bytes(1, case.n, case.k, case.bits, case.block_size, True, True)
    median = statistics.median(samples)
    return {"value": nbytes / median / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "threading": threading_kind,
            "sample": f"{calls} calls of the full M=1 K=4096 N=14336 workload, median of per-call times",
            "ms_per_call": median * 1e3}


def run_reference(args, rank: int) -> None:
    """The reference arm: the CPU implementation of this path on the host cores. The reference
    project has no MatMulNBits kernel, so this is the CPU restatement (kind "port"), its column
    panels dispatched through the reference's ExecuteRanges. Loads nothing of the CUDA product."""
    if rank != 0:
        return
    from onnx_light_cpu_b200.tools import synthetic as syn
    from oracle import nbits_oracle as o

    o.build(reference=False)
    multi = args.gpus > 1
    copies = 2 if multi else 8
    case = syn.config5(1, 4) if multi else syn.config2(1)   # the full workload in both cases
    threads = o.hardware_threads()
    threading_kind = cpu_threading(o)
    call_args = (case.a, case.b, case.scales, case.zero_points, case.bias, case.n, case.k, case.bits,
                 case.block_size)
    per_call_bytes = syn.algorithmic_bytes(1, case.n, case.k, case.bits, case.block_size,
                                           case.zero_points is not None, case.bias is not None)
    # bound the run: a step is `copies` calls
    steps = max(1, min(args.steps, 10 if multi else 50))
    warmup = max(1, min(args.warmup, 3 if multi else 5))
    for _ in range(warmup):
        o.matmul_f32_fast(*call_args, threads=threads)
    start = time.perf_counter()
    for _ in range(steps * copies):
        o.matmul_f32_fast(*call_args, threads=threads)
    elapsed = time.perf_counter() - start
    value = per_call_bytes * steps * copies / elapsed / 1e9
    sample = f"{steps} steps x {copies} calls of the full workload (same weights each call)"
    line = {
        "impl": "reference", "metric": "MatMulNBits 4-bit M=1 HBM GB/s", "value": value, "unit": "GB/s",
        "n_gpus": args.gpus, "steps": steps, "warmup": warmup, "ms_per_step": elapsed / steps * 1e3,
        "higher_is_better": True, "scaling": "strong" if multi else "weak", "vs_baseline": None, "dtype": "f32",
        "data": "synthetic", "config": workload_config(multi, copies, per_call_bytes),
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": threads, "kind": "port",
                         "threading": threading_kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference ships no MatMulNBits kernel; this is the CPU restatement used as the oracle",
    }
    print(json.dumps(line), flush=True)


def time_steps(torch, dist, step, steps: int, warmup: int, world: int) -> float:
    """Seconds for exactly `steps` calls of step(), device-timed, max over ranks."""
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    begin = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    begin.record()
    for _ in range(steps):
        step()
    end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    seconds = begin.elapsed_time(end) / 1e3
    if world > 1:
        t = torch.tensor([seconds], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        seconds = float(t.item())
    return seconds


def capture_graph(torch, step):
    """Captures step() into a CUDA graph; returns a replay callable (or step on failure)."""
    try:
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            step()
        torch.cuda.current_stream().wait_stream(stream)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step()
        return graph.replay, True
    except Exception as exc:  # pragma: no cover - depends on the driver
        print(f"bench: CUDA graph capture failed ({exc}); timing plain launches", file=sys.stderr)
        torch.cuda.synchronize()
        return step, False


def device_weights(torch, pkg, m_cfg: dict, copies: int, seed: int, zp: bool, bias: bool):
    """`copies` random weight sets resident on the device (generated there, same distributions
    as the synthetic configurations) and their handles."""
    gen = torch.Generator(device="cuda")
    gen.manual_seed(seed)
    k, n, bits, bs = m_cfg["k"], m_cfg["n"], m_cfg["bits"], m_cfg["block_size"]
    nb = -(-k // bs)
    out = []
    for _ in range(copies):
        b = torch.randint(0, 256, (n, nb, bs * bits // 8), dtype=torch.uint8, device="cuda", generator=gen)
        scales = (torch.randn(n * nb, device="cuda", generator=gen).abs() * 0.01).float()
        zero_points = (torch.randint(0, 256, (n, (nb * bits + 7) // 8), dtype=torch.uint8, device="cuda",
                                     generator=gen) if zp else None)
        bias_t = (torch.randn(n, device="cuda", generator=gen) * 0.1).float() if bias else None
        out.append(pkg.MatMulNBitsWeights(b, scales, zero_points, bias_t, K=k, N=n, bits=bits, block_size=bs))
    return out


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=200)
    parser.add_argument("--warmup", type=int, default=20)
    parser.add_argument("--impl", default="b200", choices=["b200", "reference"])
    parser.add_argument("--skip-extras", action="store_true", help="headline only (used for profiling runs)")
    parser.add_argument("--no-graph", action="store_true", help="plain launches instead of a CUDA graph")
    parser.add_argument("--gather", default="peer", choices=["peer", "nccl"],
                        help="multi-GPU: kernels store into every rank's result through peer-mapped memory "
                             "(default) or an NCCL all-gather follows each kernel")
    parser.add_argument("--decode-path", default="auto", choices=["auto", "gemv", "mma", "imma", "direct", "resident"],
                        help="kernel family for the decode workload (auto = library dispatch)")
    args = parser.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import torch
    import torch.distributed as dist

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from onnx_light_cpu_b200 import build

    if rank == 0:
        build.build_all()
    if world > 1:
        dist.barrier()
    import onnx_light_cpu_b200 as pkg
    from onnx_light_cpu_b200 import _capi
    from onnx_light_cpu_b200.matmul_nbits import _ptr  # noqa: F401

    _capi.load()
    peaks, peak_kind = measured_peaks()
    multi = world > 1
    extras: dict = {}

    if not multi:
        cfg = DECODE
        copies = 8
        weights = device_weights(torch, pkg, cfg, copies, seed=1201, zp=True, bias=True)
        m = 1
        a = torch.randn(m, cfg["k"], device="cuda").half().float()
        ys = [torch.empty(m, cfg["n"], device="cuda") for _ in range(copies)]
        per_launch_bytes = weights[0].algorithmic_bytes(m)
        assert copies * per_launch_bytes > L2_BYTES

        decode_path = {"auto": _capi.PATH_AUTO, "gemv": _capi.PATH_GEMV, "mma": _capi.PATH_GEMV_MMA,
                       "imma": _capi.PATH_GEMV_IMMA, "direct": _capi.PATH_GEMV_DIRECT,
                       "resident": _capi.PATH_GEMV_RESIDENT}[args.decode_path]

        def step():
            for w, y in zip(weights, ys):
                w.matmul_device(a, y, path=decode_path)

        step()
        torch.cuda.synchronize()
        kernel_name = _capi.last_kernel()
        if any(w.poll_status() != 0 for w in weights):
            raise SystemExit(f"bench: {kernel_name} reported a device-side timeout; not timing a broken kernel")
        replay, graphed = (step, False) if args.no_graph else capture_graph(torch, step)
        launches_before = _capi.launch_count()
        with ClockSampler(local_rank) as clocks:
            seconds = time_steps(torch, dist, replay, args.steps, args.warmup, world)
            clocks.hold(replay, torch)
        # graph replays do not pass through the launcher: count the kernels inside the graph
        gpu_launches = args.steps * copies if graphed else _capi.launch_count() - launches_before
        value = per_launch_bytes * copies * args.steps / seconds / 1e9
        launch_us = seconds / (args.steps * copies) * 1e6
        config = workload_config(False, copies, per_launch_bytes)
        details = {"cuda_graph": graphed, "kernel": kernel_name}
        roofline = {"bound": "hbm", "achieved": value, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": value / peaks["hbm_gbs"], "traffic": NCU_DECODE_TRAFFIC_BYTES.get(kernel_name),
                    "traffic_source": "constant from one ncu capture of this kernel on this workload, not this run",
                    "peak_kind": f"of {peak_kind} (copy bandwidth)", "kernel": kernel_name,
                    "us_per_launch": launch_us, "algorithmic_bytes_per_launch": per_launch_bytes}
        scaling = "weak"

        # ---- end to end through the host-buffer call ----
        a_host = a.cpu().pin_memory()
        y_host = torch.empty(m, cfg["n"]).pin_memory()
        host_steps = max(3, min(args.steps, 50))

        a_pointer, y_pointer = a_host.data_ptr(), y_host.data_ptr()

        def host_step():
            for w in weights:
                w.matmul_host_ptr(a_pointer, m, y_pointer)

        for _ in range(3):
            host_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(host_steps):
            host_step()
        host_seconds = time.perf_counter() - t0
        e2e = {"value": per_launch_bytes * copies * host_steps / host_seconds / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": copies * a_host.numel() * 4, "d2h_bytes_per_step": copies * y_host.numel() * 4,
               "us_per_call": host_seconds / (host_steps * copies) * 1e6,
               "note": "constant weights resident on the device (uploaded once per node); A and Y are pinned host buffers"}

        if not args.skip_extras:
            # ---- decode sweep M = 4, 16 ----
            sweep = {}
            for m_sweep in (4, 8, 16):
                a_s = torch.randn(m_sweep, cfg["k"], device="cuda").half().float()
                ys_s = [torch.empty(m_sweep, cfg["n"], device="cuda") for _ in range(copies)]

                def sweep_step():
                    for w, y in zip(weights, ys_s):
                        w.matmul_device(a_s, y, path=decode_path)

                sweep_step()
                torch.cuda.synchronize()
                name = _capi.last_kernel()
                rep, _ = capture_graph(torch, sweep_step)
                sec = time_steps(torch, dist, rep, max(5, args.steps // 4), 3, 1)
                nbytes = weights[0].algorithmic_bytes(m_sweep)
                gbs = nbytes * copies * max(5, args.steps // 4) / sec / 1e9
                sweep[f"m{m_sweep}"] = {"gbs": gbs, "frac_of_hbm_peak": gbs / peaks["hbm_gbs"], "kernel": name}
            extras["decode_sweep"] = sweep
            del weights, ys
            torch.cuda.empty_cache()

            # ---- accuracy_level 4 (int8 activations, integer MMA), cfg4 gate/up geometry, M = 16 ----
            icfg = {"k": 4096, "n": 14336, "bits": 4, "block_size": 32}
            icopies = 5
            iw = device_weights(torch, pkg, icfg, icopies, seed=1401, zp=False, bias=False)
            a_i8 = torch.randn(16, icfg["k"], device="cuda")
            ys_i8 = [torch.empty(16, icfg["n"], device="cuda") for _ in range(icopies)]

            def int8_step():
                for w, y in zip(iw, ys_i8):
                    w.matmul_device(a_i8, y, accuracy_level=4)

            int8_step()
            torch.cuda.synchronize()
            iname = _capi.last_kernel()
            istatus = max(w.poll_status() for w in iw)
            rep, _ = capture_graph(torch, int8_step)
            isteps = max(5, args.steps // 4)
            sec = time_steps(torch, dist, rep, isteps, 3, 1)
            ibytes = iw[0].algorithmic_bytes(16)
            igbs = ibytes * icopies * isteps / sec / 1e9
            extras["int8"] = {
                "workload": "cfg4 gate/up projection M=16 K=4096 N=14336 bits=4 block=32, accuracy_level=4",
                "gbs": igbs, "frac_of_hbm_peak": igbs / peaks["hbm_gbs"], "us_per_call": sec / (icopies * isteps) * 1e6,
                "kernel": iname, "device_status": istatus,
                "includes": "activation quantization kernel + integer-MMA kernel (dependent launch)"}
            # ---- same projection at accuracy_level 0: digit rows through the integer-MMA kernel ----
            def level0_step():
                for w, y in zip(iw, ys_i8):
                    w.matmul_device(a_i8, y)

            level0_step()
            torch.cuda.synchronize()
            lname = _capi.last_kernel()
            lstatus = max(w.poll_status() for w in iw)
            rep, _ = capture_graph(torch, level0_step)
            sec = time_steps(torch, dist, rep, isteps, 3, 1)
            lgbs = ibytes * icopies * isteps / sec / 1e9
            extras["level0_m16_block32"] = {
                "workload": "cfg4 gate/up projection M=16 K=4096 N=14336 bits=4 block=32, accuracy_level=0",
                "gbs": lgbs, "frac_of_hbm_peak": lgbs / peaks["hbm_gbs"], "us_per_call": sec / (icopies * isteps) * 1e6,
                "kernel": lname, "device_status": lstatus,
                "includes": "digit rows of both K slices + one-pass integer-MMA kernel over 48 digit rows + sum of the slices"}
            del iw, ys_i8
            torch.cuda.empty_cache()

            # ---- 8-bit weights, M = 8: one column shard of the large-N projection, digit columns on integer MMA ----
            ucfg = {"k": 4096, "n": 16032, "bits": 8, "block_size": 32}
            ucopies = 4
            uw = device_weights(torch, pkg, ucfg, ucopies, seed=1501, zp=True, bias=False)
            a_u8 = torch.randn(8, ucfg["k"], device="cuda")
            ys_u8 = [torch.empty(8, ucfg["n"], device="cuda") for _ in range(ucopies)]

            def u8_step():
                for w, y in zip(uw, ys_u8):
                    w.matmul_device(a_u8, y)

            u8_step()
            torch.cuda.synchronize()
            uname = _capi.last_kernel()
            ustatus = max(w.poll_status() for w in uw)
            rep, _ = capture_graph(torch, u8_step)
            sec = time_steps(torch, dist, rep, isteps, 3, 1)
            ubytes = uw[0].algorithmic_bytes(8)
            ugbs = ubytes * ucopies * isteps / sec / 1e9
            extras["u8_shard_m8"] = {
                "workload": "cfg5 column shard M=8 K=4096 N=16032 bits=8 block=32 zp, accuracy_level=0",
                "gbs": ugbs, "frac_of_hbm_peak": ugbs / peaks["hbm_gbs"], "us_per_call": sec / (ucopies * isteps) * 1e6,
                "kernel": uname, "device_status": ustatus,
                "includes": "digit kernel + integer-MMA kernel (dependent launch)"}
            del uw, ys_u8
            torch.cuda.empty_cache()

            # ---- sibling nodes in one call: gate + up of the decode workload, M = 1, one launch per pair ----
            from onnx_light_cpu_b200.matmul_nbits import matmul_device_group
            pairs = 4
            gw = device_weights(torch, pkg, cfg, 2 * pairs, seed=1211, zp=True, bias=True)
            gy = [torch.empty(1, cfg["n"], device="cuda") for _ in range(2 * pairs)]
            a_g = torch.randn(1, cfg["k"], device="cuda").half().float()

            def group_step():
                for i in range(pairs):
                    matmul_device_group(gw[2 * i:2 * i + 2], a_g, gy[2 * i:2 * i + 2])

            group_step()
            torch.cuda.synchronize()
            gname = _capi.last_kernel()
            gstatus = max(w.poll_status() for w in gw)
            rep, _ = capture_graph(torch, group_step)
            gsteps = max(5, args.steps // 2)
            sec = time_steps(torch, dist, rep, gsteps, 3, 1)
            gbytes = gw[0].algorithmic_bytes(1)
            ggbs = gbytes * 2 * pairs * gsteps / sec / 1e9
            extras["group_gate_up_m1"] = {
                "workload": "two M=1 K=4096 N=14336 bits=4 block=128 zp+bias nodes that share A, one call per pair",
                "gbs": ggbs, "frac_of_hbm_peak": ggbs / peaks["hbm_gbs"],
                "us_per_pair": sec / (pairs * gsteps) * 1e6, "us_per_node": sec / (2 * pairs * gsteps) * 1e6,
                "kernel": gname, "launches_per_pair": 1, "device_status": gstatus}
            del gw, gy
            torch.cuda.empty_cache()

            # ---- the seven projections of a decoder layer (cfg4), M = 16, both accuracy levels ----
            from onnx_light_cpu_b200.tools.decoder_layer import DecoderLayerProjections
            layers = [DecoderLayerProjections.synthetic(16, 0) for _ in range(2)]   # 2 x 136 MB > L2
            layer_inputs = [layer.inputs_from_cases() for layer in layers]
            layer_bytes = layers[0].algorithmic_bytes(16)
            layer_extra = {"workload": "cfg4 decoder layer: q k v o gate up down, M=16 bits=4 block=32, "
                                       "q/k/v and gate/up as grouped calls",
                           "algorithmic_bytes": layer_bytes, "layers_rotated": len(layers)}
            for level in (0, 4):
                for grouped in (True, False):
                    def layer_step():
                        for layer, inputs in zip(layers, layer_inputs):
                            layer.run(inputs, accuracy_level=level, grouped=grouped)

                    before = _capi.launch_count()
                    layer_step()
                    torch.cuda.synchronize()
                    launches = (_capi.launch_count() - before) // len(layers)
                    lstatus = max(layer.poll_status() for layer in layers)
                    rep, _ = capture_graph(torch, layer_step)
                    lsteps = max(5, args.steps // 4)
                    sec = time_steps(torch, dist, rep, lsteps, 3, 1)
                    us = sec / (len(layers) * lsteps) * 1e6
                    layer_extra[f"level{level}" + ("" if grouped else "_node_by_node")] = {
                        "us_per_layer": us, "gbs": layer_bytes / us / 1e3,
                        "frac_of_hbm_peak": layer_bytes / us / 1e3 / peaks["hbm_gbs"],
                        "launches_per_layer": launches, "device_status": lstatus}
            extras["layer_cfg4"] = layer_extra
            for layer in layers:
                layer.close()
            del layers, layer_inputs
            torch.cuda.empty_cache()

            # ---- prefill M = 2048 and M = 8192 (bf16 tcgen05 path) ----
            pw = device_weights(torch, pkg, PREFILL, 1, seed=1301, zp=True, bias=False)[0]
            for pm, key in ((PREFILL["m"], "prefill"), (8192, "prefill_m8192")):
                sets = 3 if pm <= 2048 else 2  # rotate A/Y so that A + Y + weights exceed L2 between repeats
                a_p = [torch.randn(pm, PREFILL["k"], device="cuda") for _ in range(sets)]
                y_p = [torch.empty(pm, PREFILL["n"], device="cuda") for _ in range(sets)]

                def prefill_step():
                    for a_i, y_i in zip(a_p, y_p):
                        pw.matmul_device(a_i, y_i)

                prefill_step()
                torch.cuda.synchronize()
                pname = _capi.last_kernel()
                status = pw.poll_status()
                psteps = max(5, args.steps // 10)
                prefill_replay, _ = capture_graph(torch, prefill_step)
                # events around the whole call: the fp32->bf16 activation pre-pass is inside
                sec = time_steps(torch, dist, prefill_replay, psteps, 3, 1)
                flops = 2.0 * pm * PREFILL["n"] * PREFILL["k"]
                tflops = flops * sets * psteps / sec / 1e12
                extras[key] = {
                    "workload": f"cfg3 prefill M={pm} K=4096 N=4096 bits=4 block=64 zp",
                    "tflops": tflops, "us_per_call": sec / (sets * psteps) * 1e6, "kernel": pname,
                    "device_status": status,
                    "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                                 "frac": tflops / peaks["bf16_tflops"],
                                 "frac_of_sustained": tflops / peaks["bf16_tflops_sustained"],
                                 "peak_kind": f"of {peak_kind} (cuBLAS bf16 burst)", "traffic": None},
                    "includes": "fp32->bf16 activation pre-pass + GEMM kernel, replayed from a CUDA graph"}
                del a_p, y_p, prefill_replay
                torch.cuda.empty_cache()
            del pw
    else:
        # ---- multi-GPU: column-sharded lm-head, NCCL all-gather of the output columns ----
        cfg = dict(LMHEAD)
        if cfg["n"] % world != 0:
            raise SystemExit("N must divide by the number of GPUs")
        shard_cfg = dict(cfg, n=cfg["n"] // world)
        copies = 2
        weights = device_weights(torch, pkg, shard_cfg, copies, seed=1500 + rank, zp=True, bias=False)
        m = 1
        a = torch.randn(m, cfg["k"], device="cuda")
        dist.broadcast(a, src=0)
        full_bytes = _capi.algorithmic_bytes(m, cfg["n"], cfg["k"], cfg["bits"], cfg["block_size"], True, False)
        from onnx_light_cpu_b200.tools import sharded

        gather = None
        if args.gather == "peer":
            # one kernel per node: it stores this rank's columns into all ranks' gathered results
            # and a one-warp kernel behind it exchanges "done" flags (no collective on the data path)
            try:
                gather = sharded.PeerGather(dist, local_rank, m_max=m, n_shard=shard_cfg["n"], slots=copies)
                gather.run(weights[0], a, 0)   # one step: every rank sees whether the path works here
                torch.cuda.synchronize()
                works = 1 if weights[0].poll_status() == 0 else 0
            except Exception as exc:  # pragma: no cover - depends on the box
                print(f"bench: peer-store gather unavailable on rank {rank} ({exc}); using NCCL", file=sys.stderr)
                works = 0
            flag = torch.tensor([works], device="cuda")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            if int(flag.item()) == 0:   # all ranks take the same path
                gather = None
                args.gather = "nccl"
        if gather is not None:
            y_full = [gather.result(i) for i in range(copies)]

            def step():
                # every node pushes its columns to the peers and publishes "stored" from its own last
                # CTA; only the step's last node then waits for the other ranks' flags (seeing a rank's
                # flag of a node implies its earlier nodes: every rank runs the nodes in this order)
                for i, w in enumerate(weights):
                    gather.run(w, a, i, wait=(i == copies - 1))
        else:
            y_shard = [torch.empty(m, shard_cfg["n"], device="cuda") for _ in range(copies)]
            y_full = [torch.empty(world, m, shard_cfg["n"], device="cuda") for _ in range(copies)]

            def step():
                for w, ys_, yf in zip(weights, y_shard, y_full):
                    w.matmul_device(a, ys_)
                    dist.all_gather_into_tensor(yf, ys_)

        step()
        torch.cuda.synchronize()
        kernel_name = _capi.last_kernel()
        # ---- before any timing: the gathered result of one step against every rank's own product ----
        # Rank r's columns must sit in slot [r, :, :] of the gathered result on EVERY rank. Each rank
        # computes its shard once more into plain local memory, the shards travel over an all-gather,
        # and every rank compares its gathered buffers with them, value by value.
        own = torch.empty(m, shard_cfg["n"], device="cuda")
        mismatch = 0
        for i, w in enumerate(weights):
            w.matmul_device(a, own)
            expected = torch.empty(world, m, shard_cfg["n"], device="cuda")
            dist.all_gather_into_tensor(expected, own)
            torch.cuda.synchronize()
            if not torch.equal(expected, y_full[i][:, :m, :]):
                mismatch += 1
        bad = torch.tensor([mismatch], device="cuda")
        dist.all_reduce(bad, op=dist.ReduceOp.SUM)
        if int(bad.item()) != 0:
            raise SystemExit(f"bench: gathered result differs from the ranks' own products ({int(bad.item())} buffers)")
        gather_checked = True
        # The peer-store step is kernels only and replays from a CUDA graph. With NCCL the pair is
        # launched per step: capturing kernel + all-gather did not complete on this stack.
        if gather is not None and not args.no_graph:
            replay, graphed = capture_graph(torch, step)
            ok = torch.tensor([1 if graphed else 0], device="cuda")
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            if int(ok.item()) == 0:
                raise SystemExit("bench: CUDA graph capture of the peer-store step failed on some rank")
        else:
            replay, graphed = step, False
        launches_before = _capi.launch_count()
        with ClockSampler(local_rank) as clocks:
            seconds = time_steps(torch, dist, replay, args.steps, args.warmup, world)
            launches_timed = args.steps * copies if graphed else _capi.launch_count() - launches_before
            clocks.hold(replay, torch)
        gpu_launches = launches_timed * world
        value = full_bytes * copies * args.steps / seconds / 1e9
        how = ("peer stores, flag publish and the step's one flag wait inside the nodes' kernels"
               if gather is not None else "NCCL all-gather")
        config = workload_config(True, copies, full_bytes)
        details = {"shard_columns": shard_cfg["n"], "gathered_layout": "[ranks, M, N/ranks]", "kernel": kernel_name,
                   "cuda_graph": graphed, "gather": args.gather, "gather_how": how, "gather_checked": gather_checked}
        shard_bytes = weights[0].algorithmic_bytes(m)
        roofline = {"bound": "hbm", "achieved": value / world, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": value / world / peaks["hbm_gbs"], "traffic": None,
                    "peak_kind": f"of {peak_kind} (copy bandwidth), per GPU, gather time included",
                    "algorithmic_bytes_per_launch": shard_bytes}
        scaling = "strong"
        # end to end: A from pinned host memory, gathered Y back to pinned host memory
        a_host = a.cpu().pin_memory()
        y_host = torch.empty(world, m, shard_cfg["n"]).pin_memory()
        host_steps = max(3, min(args.steps, 50))

        def host_step():
            for i, w in enumerate(weights):
                a.copy_(a_host, non_blocking=True)
                if gather is not None:
                    gather.run(w, a, i)
                else:
                    w.matmul_device(a, y_shard[i])
                    dist.all_gather_into_tensor(y_full[i], y_shard[i])
                y_host.copy_(y_full[i], non_blocking=True)
                torch.cuda.synchronize()

        host_step()
        dist.barrier()
        t0 = time.perf_counter()
        for _ in range(host_steps):
            host_step()
        dist.barrier()
        host_seconds = time.perf_counter() - t0
        e2e = {"value": full_bytes * copies * host_steps / host_seconds / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": copies * a_host.numel() * 4, "d2h_bytes_per_step": copies * y_host.numel() * 4}

        if not args.skip_extras:
            # ---- the other sizes of the configuration through the same gathered path: M in {8, 256},
            # 8-bit weights (shapes the decode kernels do not take run through the ordinary dispatch
            # and one kernel that copies the local window to the peers) ----
            if gather is not None:
                for key, m_x, bits_x in (("lmhead_m8", 8, 4), ("lmhead_m256", 256, 4), ("lmhead_bits8_m1", 1, 8),
                                         ("lmhead_bits8_m8", 8, 8)):
                    cfg_x = dict(shard_cfg, bits=bits_x)
                    w_x = weights if bits_x == cfg["bits"] else device_weights(torch, pkg, cfg_x, copies,
                                                                               seed=1580 + rank, zp=True, bias=False)
                    gather_x = sharded.PeerGather(dist, local_rank, m_max=m_x, n_shard=shard_cfg["n"], slots=copies)
                    a_x = torch.randn(m_x, cfg["k"], device="cuda")
                    dist.broadcast(a_x, src=0)

                    def step_x():
                        for i, w in enumerate(w_x):
                            gather_x.run(w, a_x, i, wait=(i == copies - 1))

                    step_x()
                    torch.cuda.synchronize()
                    name_x = _capi.last_kernel()
                    # the gathered values against the ranks' own products, as for the headline
                    own_x = torch.empty(m_x, shard_cfg["n"], device="cuda")
                    w_x[0].matmul_device(a_x, own_x)
                    expected_x = torch.empty(world, m_x, shard_cfg["n"], device="cuda")
                    dist.all_gather_into_tensor(expected_x, own_x)
                    torch.cuda.synchronize()
                    # (the gathered path and the plain call may pick different kernels: compare to 2e-5)
                    worst_x = float((expected_x - gather_x.result(0)).abs().max() / expected_x.abs().max())
                    same_x = torch.tensor([1 if worst_x <= 2e-5 else 0], device="cuda")
                    dist.all_reduce(same_x, op=dist.ReduceOp.MIN)
                    rep_x, graphed_x = capture_graph(torch, step_x)
                    ok_x = torch.tensor([1 if graphed_x else 0], device="cuda")
                    dist.all_reduce(ok_x, op=dist.ReduceOp.MIN)
                    if int(ok_x.item()) == 1:
                        steps_x = max(5, args.steps // 4)
                        sec_x = time_steps(torch, dist, rep_x, steps_x, 3, world)
                        bytes_x = _capi.algorithmic_bytes(m_x, cfg["n"], cfg["k"], bits_x, cfg["block_size"], True, False)
                        extras[key] = {"gbs": bytes_x * copies * steps_x / sec_x / 1e9,
                                       "us_per_node": sec_x / (copies * steps_x) * 1e6, "kernel": name_x,
                                       "gather_checked": bool(int(same_x.item())),
                                       "workload": f"cfg5 lm-head M={m_x} bits={bits_x}, same shards and gather"}
                        if m_x >= 64:
                            extras[key]["tflops"] = 2.0 * m_x * cfg["n"] * cfg["k"] * copies * steps_x / sec_x / 1e12
                    torch.cuda.synchronize()
                    dist.barrier()
                    gather_x.close()
                    if w_x is not weights:
                        del w_x
                    del a_x, own_x, expected_x
                    torch.cuda.empty_cache()
            # ---- like-for-like base of the scaling curve: the same node, unsharded, on one GPU ----
            # Timed by rank 0 alone in this very run (337 MB of operands fit); the other ranks wait.
            del weights
            torch.cuda.empty_cache()
            dist.barrier()
            if rank == 0:
                base_w = device_weights(torch, pkg, cfg, copies, seed=1499, zp=True, bias=False)
                base_y = [torch.empty(m, cfg["n"], device="cuda") for _ in range(copies)]

                def base_step():
                    for w, y in zip(base_w, base_y):
                        w.matmul_device(a, y)

                base_step()
                torch.cuda.synchronize()
                base_name = _capi.last_kernel()
                base_rep, _ = capture_graph(torch, base_step)
                base_steps = max(5, args.steps // 4)
                base_sec = time_steps(torch, dist, base_rep, base_steps, 3, 1)
                extras["scaling_base"] = {
                    "workload": "cfg5 lm-head M=1 K=4096 N=128256 bits=4 block=32 zp, unsharded on one GPU",
                    "value": full_bytes * copies * base_steps / base_sec / 1e9, "unit": "GB/s",
                    "us_per_node": base_sec / (copies * base_steps) * 1e6, "kernel": base_name,
                    "note": "divide `value` of this line by this value for the like-for-like speed-up over one GPU"}
                del base_w, base_y
            dist.barrier()

    if rank == 0:
        line = {
            "metric": "MatMulNBits 4-bit M=1 HBM GB/s", "value": value, "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": seconds / args.steps * 1e3,
            "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": config, "details": details, "roofline": roofline, "e2e": e2e,
            "gpu_launches": int(gpu_launches), "clocks": clocks.summary(),
        }
        line.update(extras)
        if not multi and not args.skip_extras:
            line["cpu_baseline"] = cpu_port_baseline()
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
