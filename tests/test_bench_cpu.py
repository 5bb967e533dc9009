"""bench.py's host-side pieces, without a GPU: the algorithmic bytes and flops behind the roofline figures, and the
parsing of the clock poller's lines with the timed window."""
import datetime
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)

from c0ven_b200 import synth  # noqa: E402


def test_algorithmic_work_of_the_headline_batch():
    w = dict(synth.CONFIGS["ragged3521_q4_k_zipf"], name="ragged3521_q4_k_zipf")
    a = bench.algorithmic(w, 3521, 161)
    # a routed assignment: gate and up 2 * 2 * 2048 * 512 flops, down 2 * 2048 * 512
    assert a["flops_gate_up"] == 3521 * 10 * 4_194_304
    assert a["flops_down"] == 3521 * 10 * 2_097_152
    # an expert's gate and up in Q4_K: 2 * 512 rows * 1152 bytes; down: 2048 rows * 288 bytes
    assert a["bytes_gate_up"] == 161 * 2 * 512 * 1152
    assert a["bytes_down"] == 161 * 2048 * 288
    assert a["bytes_layer"] == 513 * 2048 * 4 + 161 * 1_769_472 + 1_769_472 + 2 * 3521 * 2048 * 4


def test_clock_lines_inside_the_window_only():
    s = bench.ClockSampler(None)
    t0 = datetime.datetime(2026, 1, 2, 3, 4, 5).timestamp()

    def line(dt, sm, slow="Not Active"):
        ts = datetime.datetime.fromtimestamp(t0 + dt).strftime("%Y/%m/%d %H:%M:%S.%f")[:-3]
        return f"{ts}, 0, {sm}, 1965, 500.0, 0x0, {slow}, Not Active, Not Active, Not Active\n"

    s.lines = [line(-5.0, 300, "Active"), line(0.1, 1900), line(0.2, 1950), line(9.0, 400)]
    s.window(t0, t0 + 0.5)
    got = s.summary()
    assert got["samples"] == 2 and got["sm_mhz"] == 1925.0 and got["sm_max_mhz"] == 1965.0 and got["reasons"] == []
    s.window(t0 + 100, t0 + 101)  # nothing inside: every sample counts, the slowdown too
    got = s.summary()
    assert got["samples"] == 4 and got["reasons"] == ["hw_slowdown"]
