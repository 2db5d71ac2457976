"""The benchmark's vectorised fp8 quantiser produces the same code bytes as the reference's RNE cast
(so the fp8 GEMM inputs are what the configuration describes: N(0,1) scaled to amax = max finite, RNE)."""
import numpy as np

from intel_gaudi3_software_b200 import abi, workloads as bench


def test_quantiser_matches_oracle(port):
    rng = np.random.default_rng(0)
    v = rng.standard_normal(200000).astype(np.float32)
    v[:64] = np.float32(2.0) ** -np.arange(64, dtype=np.float32) * v[0]   # reach the denormal range
    for dtype, ew, bias, mode, mx in ((abi.FP8_143, 4, 7, abi.INFNAN_MINIMAL, 448.0), (abi.FP8_152, 5, 15, abi.INFNAN_FULL, 57344.0)):
        got = bench.quantise_fp8(v, dtype, bias)
        scaled = v * np.float32(mx / np.abs(v).max())
        want = port.fp32_to_fp8(scaled, ew, bias, abi.RM_NE, None, False, False, False, False, mode)
        assert (got == want).all(), (dtype, int((got != want).sum()))


def test_workload_counts_match_the_configurations():
    f, b = bench.workload_counts(bench.WORKLOADS["fp8_gemm_8192"])
    assert f == 2.0 * 8192**3 and b == 2 * 8192 * 8192 + 2 * 8192 * 8192
    f, b = bench.workload_counts(bench.WORKLOADS["conv_fwd"])
    assert abs(f - 2.3676e11) / 2.3676e11 < 1e-3 and abs(b - 2.067e8) / 2.067e8 < 1e-3
    f, b = bench.workload_counts(bench.WORKLOADS["fp8_bgemm_attn"])
    assert abs(f - 2.7488e11) / 2.7488e11 < 1e-3 and abs(b - 2.2146e9) / 2.2146e9 < 1e-3
