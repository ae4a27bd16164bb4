"""Pure-function tests of the measurement tools (no GPU, no heavy dependencies), in the style of
the reference's unittests/python/test_integer_gemm_parity_benchmark.py."""

from onnx_light_cpu_b200.tools import benchmark_nbits_parity as parity
from onnx_light_cpu_b200.tools import nbits_throughput as thr


def test_repeat_count_is_clamped():
    assert thr.repeats_for(1.0) == 5
    assert thr.repeats_for(1e-9) == 101
    assert thr.repeats_for(0.0) == 101
    assert thr.repeats_for(0.001) == 20


def test_weight_copies_defeat_l2():
    assert thr.copies_for(31_555_584) * 31_555_584 > thr.L2_BYTES
    assert thr.copies_for(10 ** 9) == 1
    assert thr.copies_for(1) == 16


def test_summaries_keep_raw_samples_and_use_the_median():
    s = thr.summarize([5.0, 1.0, 3.0, 2.0, 4.0, 100.0, 6.0])
    assert s["median"] == 4.0 and s["min"] == 1.0 and s["max"] == 100.0 and len(s["samples"]) == 7
    assert s["iqr"] > 0
    assert parity.stats([3.0, 1.0, 2.0])["median"] == 2.0


def test_speed_gate():
    assert parity.speed_gate([1.2, 0.95, 3.0])["passed"]
    assert not parity.speed_gate([1.2, 0.85, 3.0])["passed"]      # slowest case under 0.9
    assert not parity.speed_gate([0.95, 0.95, 0.99])["passed"]    # median under 1.0
    assert not parity.speed_gate([])["passed"]


def test_alternating_measurement_rotates_the_order():
    calls = []
    a, b = parity.measure_alternating(lambda: calls.append("a"), lambda: calls.append("b"), iterations=4, warmup=1)
    assert len(a) == len(b) == 4
    assert calls == ["a", "b", "a", "b", "b", "a", "a", "b", "b", "a"]


def test_shape_lists_cover_the_configurations():
    names = [s[0] for s in thr.SHAPES]
    assert any(n.startswith("cfg1") for n in names) and any("cfg3_prefill_m2048" == n for n in names)
    assert all(len(s) == 9 for s in thr.SHAPES) and all(len(c) == 10 for c in parity.CORPUS)
