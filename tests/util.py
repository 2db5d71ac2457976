"""Shared helpers of the test-suite: seeded inputs in the reference's formats, decoders, and the
comparison rules of the parity tests.

Tolerances (stated here once, used by every accumulation test):
  * fp32 accumulators: |gpu - ref| <= ACC_TOL * sum_k |a_k * b_k| per element (1e-5, the north
    star's "<= 1e-5 relative error on fp32 accumulators", taken norm-wise because the reference's
    own truncating accumulation sits up to ~1e-6 * sum|ab| away from the exact dot product);
  * rounded outputs: bit-exact, or at most 1 ulp of the output type, or (near cancellation, where
    an accumulator difference of 1e-5 * sum|ab| spans many ulps of a tiny result) within the
    accumulator tolerance.
"""
import numpy as np

from intel_gaudi3_software_b200 import abi, workloads

ACC_TOL = 1e-5


bf16_to_f32 = workloads.bf16_to_f32
f32_to_bf16_rne = workloads.f32_to_bf16_rne


def decode(arr, dtype, bias=0, mode=0, oracle=None):
    if dtype == abi.BF16:
        return bf16_to_f32(arr)
    if dtype in (abi.FP8_143, abi.FP8_152):
        assert oracle is not None
        return oracle.fp8_to_fp32(np.asarray(arr, dtype=np.uint8), 4 if dtype == abi.FP8_143 else 5, bias, mode)
    return np.asarray(arr, dtype=np.float32)


def gen_bf16(rng, n, dist="uniform", scale=1.0):
    v = rng.uniform(-1, 1, n) if dist == "uniform" else rng.normal(0, scale, n)
    return f32_to_bf16_rne(v.astype(np.float32))


def gen_fp8(rng, n, oracle, dtype=abi.FP8_143, bias=7, mode=abi.INFNAN_MINIMAL, amax_target=None):
    """N(0,1) scaled so that amax lands on the format's largest finite value, RNE-cast (the fp8 8192^3 GEMM configuration)."""
    v = rng.normal(0, 1, n).astype(np.float32)
    ew = 4 if dtype == abi.FP8_143 else 5
    if amax_target is None:
        if dtype == abi.FP8_143:
            amax_target = (448.0 if mode != 0 else 240.0) * 2.0 ** (7 - bias)
        else:
            amax_target = 57344.0 * 2.0 ** (15 - bias)
    v *= np.float32(amax_target / np.abs(v).max())
    return oracle.fp32_to_fp8(v, ew, bias, abi.RM_NE, None, False, True, False, False, mode)


def sum_abs_products(a_f32, b_f32):
    """sum_k |a_ik| |b_kj| in float64: the scale of the accumulation tolerance."""
    return np.abs(a_f32.astype(np.float64)) @ np.abs(b_f32.astype(np.float64))


def acc_error(gpu, ref, sabs):
    """max over elements of |gpu-ref| / sum|ab| (elements with sum|ab| == 0 must match exactly)."""
    g, r = gpu.astype(np.float64), ref.astype(np.float64)
    both_nan = np.isnan(g) & np.isnan(r)
    d = np.abs(g - r)
    d[both_nan] = 0
    d[(g == r)] = 0  # equal infinities
    with np.errstate(divide="ignore", invalid="ignore"):
        rel = np.where(sabs > 0, d / sabs, np.where(d == 0, 0.0, np.inf))
    return float(np.nanmax(rel)) if rel.size else 0.0


def ulp_diff_bits(a_bits, b_bits, width):
    """Distance in representable values between two sign-magnitude bit patterns of `width` bits."""
    a = np.asarray(a_bits).astype(np.int64)
    b = np.asarray(b_bits).astype(np.int64)
    sign = 1 << (width - 1)
    ai = np.where(a & sign, -(a & (sign - 1)), a & (sign - 1))
    bi = np.where(b & sign, -(b & (sign - 1)), b & (sign - 1))
    return np.abs(ai - bi)


def check_rounded(gpu_bits, ref_bits, width, gpu_val, ref_val, sabs, name=""):
    """The rounded-output rule above. Returns (n_inexact, n_beyond_1ulp_but_within_acc_tol)."""
    ud = ulp_diff_bits(gpu_bits, ref_bits, width)
    inexact = int((ud != 0).sum())
    far = ud > 1
    if far.any():
        d = np.abs(gpu_val.astype(np.float64) - ref_val.astype(np.float64))
        bad = far & ~(d <= ACC_TOL * sabs)
        assert not bad.any(), "%s: %d outputs differ by more than 1 ulp and more than the accumulator tolerance" % (
            name, int(bad.sum()))
    return inexact, int(far.sum())


def clear_signs(bits, dtype):
    """The operand's bit patterns with every sign bit cleared: |value| element by element."""
    if dtype == abi.BF16:
        return np.asarray(bits, dtype=np.uint16) & np.uint16(0x7FFF)
    if dtype in (abi.FP8_143, abi.FP8_152):
        return np.asarray(bits, dtype=np.uint8) & np.uint8(0x7F)
    return np.abs(np.asarray(bits, dtype=np.float32))


def conv_sum_abs(oracle, shapes, bits, dtype, cp, op, **tensor_kw):
    """sum |a_k| |b_k| of every output of a convolution: the same operation run by the oracle on the operands'
    absolute values (its own truncation errs by ~1e-6 relative, far inside its use as the scale of ACC_TOL)."""
    T = abi.make_tensor
    xs, ws, ys = shapes
    xb, wb, yb = (clear_signs(b, dtype) for b in bits)
    shp = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[op]
    out = np.zeros(int(np.prod(shp)), np.float32)
    assert oracle.conv(T(out, abi.FP32, shp), T(xb, dtype, xs, **tensor_kw), T(wb, dtype, ws, **tensor_kw), T(yb, dtype, ys, **tensor_kw), cp, op) == 0
    return out.astype(np.float64)


def assert_acc(gpu, ref, sabs, name=""):
    """The accumulator rule: |gpu - ref| <= ACC_TOL * sum|ab| for every element."""
    err = acc_error(np.asarray(gpu).reshape(-1), np.asarray(ref).reshape(-1), np.asarray(sabs, dtype=np.float64).reshape(-1))
    assert err <= ACC_TOL, "%s: accumulator error %.3g * sum|ab| exceeds %.0e" % (name, err, ACC_TOL)
    return err


class OracleAsCalculator:
    """A CPU checker behind the calculator's method names, so that the config runner's flow (run_flow) can replay a test on
    it. Raises where the backend would."""

    def __init__(self, oracle, lfsr, poly, chip=abi.CHIP_GAUDI3):
        self.oracle, self.lfsr, self.poly, self.chip = oracle, lfsr, poly, chip

    def do_convolution(self, out, x, w, y, params, op, rm=abi.RM_NE, cast=None):
        assert cast is None and self.oracle.conv(out, x, w, y, params, op, rm, chip=self.chip) == 0

    def do_batch_gemm(self, out, x, w, op, cast=None):
        assert cast is None and self.oracle.bgemm(out, x, w, op, chip=self.chip) == 0

    def do_memory_write(self, mem, mme_out, reduction_op=abi.RED_NONE, reduction_rm=0, clip_fp=False):
        assert self.oracle.memory_write(mem, mme_out, reduction_op, reduction_rm, clip_fp, chip=self.chip) == 0

    def do_activation(self, out, acc, cast):
        rc, self.lfsr = self.oracle.activation(out, acc, cast, self.lfsr, self.poly, chip=self.chip)
        assert rc == 0
