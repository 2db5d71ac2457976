"""Host-side logic of bench.py that needs no GPU: the workload description of a line, the roofline arithmetic and its
denominators, and the clock record built from time-stamped nvidia-smi samples."""
import datetime
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
import bench  # noqa: E402
from intel_gaudi3_software_b200.workloads import WORKLOADS, workload_counts  # noqa: E402

PEAKS = dict(hbm=6459.0, bf16=1656.1, bf16_sustained=1400.0, source="measured")


def test_config_names_the_workload_and_the_sharding():
    one = bench.config_dict("fp8_gemm_8192", 1, "strong")
    assert one["workload"] == "fp8_gemm_8192" and one["shape"] == {"M": 8192, "N": 8192, "K": 8192} and "model" not in one
    assert one["scaling"] == "single GPU" and one["ranks"] == 1 and "bf16 RNE" in one["output"]
    eight = bench.config_dict("conv_dedw", 8, "strong")
    assert eight["scaling"] == "strong" and eight["ranks"] == 8 and "all-reduce" in eight["sharding"]
    assert "stochastic" in bench.config_dict("fp8_gemm_8192_sr", 1, "strong")["output"]


def test_roofline_arithmetic_and_denominators():
    wl = WORKLOADS["fp8_gemm_8192"]
    flops, alg_bytes = workload_counts(wl)
    assert flops == 2 * 8192 ** 3 and alg_bytes == 2 * 8192 * 8192 + 2 * 8192 * 8192
    # without a measured fp8 figure the denominator is twice the bf16 burst figure, and says so
    r = bench.roofline_of("fp8_gemm_8192", wl, flops, alg_bytes, 0.3665, PEAKS, None)
    assert r["bound"] == "tensor" and r["unit"] == "TFLOP/s" and abs(r["peak"] - 2 * 1656.1) < 1e-9 and r["peak_note"].startswith("2 x the measured bf16")
    assert abs(r["achieved"] - flops / 0.3665e-3 / 1e12) < 1e-6 and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-12
    assert abs(r["frac"] - 0.906) < 2e-3 and r["traffic"] == bench.NCU_TRAFFIC_BYTES["fp8_gemm_8192"]
    # with one, burst and sustained figures are kept apart
    fp8 = dict(burst=3100.0, sustained=2600.0)
    assert bench.roofline_of("fp8_gemm_8192", wl, flops, alg_bytes, 0.37, PEAKS, fp8)["peak"] == 3100.0
    s = bench.roofline_of("fp8_gemm_8192", wl, flops, alg_bytes, 0.43, PEAKS, fp8, sustained=True)
    assert s["peak"] == 2600.0 and abs(s["frac_of_2x_bf16"] - s["achieved"] / 2800.0) < 1e-12
    # the small-K batched GEMM is judged by its bytes against the copy bandwidth
    awl = WORKLOADS["fp8_bgemm_attn"]
    af, ab = workload_counts(awl)
    a = bench.roofline_of("fp8_bgemm_attn", awl, af, ab, 0.4, PEAKS, fp8)
    assert a["bound"] == "hbm" and a["unit"] == "GB/s" and a["peak"] == 6459.0 and abs(a["achieved"] - ab / 0.4e-3 / 1e9) < 1e-6
    # wide operands: tf32 runs at half the bf16 rate, fp32 as three tf32 products
    assert abs(bench.peak_for(WORKLOADS["tf32_gemm_4096"], PEAKS, None)[0] - 1656.1 / 2) < 1e-9
    assert abs(bench.peak_for(WORKLOADS["fp32_gemm_4096"], PEAKS, None)[0] - 1656.1 / 6) < 1e-9


def test_clock_record_uses_only_the_samples_inside_the_window():
    s = bench.ClockSampler.__new__(bench.ClockSampler)      # no nvidia-smi here: feed the samples by hand
    t0 = datetime.datetime(2025, 1, 1, 12, 0, 0)
    at = lambda ms: t0 + datetime.timedelta(milliseconds=ms)  # noqa: E731
    s.proc, s.windows = object(), {"timed": [at(100), at(160)], "empty": [at(500), at(501)]}
    s.samples = [(at(20 * i), 1965.0 if i < 5 else 1300.0 + i, 1965.0, 400.0 + i, [] if i < 5 else ["sw_power_cap"]) for i in range(12)]
    w = s.window("timed", ms_per_step=0.4)
    assert w["samples_under_load"] == 4 and w["sm_max_mhz"] == 1965.0 and w["reasons"] == ["sw_power_cap"]
    assert w["sm_mhz"] == 1306.5 and abs(w["window_s"] - 0.06) < 1e-9 and abs(w["ms_x_mhz"] - 0.4 * 1306.5) < 1e-9
    e = s.window("empty")
    assert e["samples_under_load"] == 0 and e["sm_mhz"] is None and e["reasons"] == []
    assert s.total() == 12
