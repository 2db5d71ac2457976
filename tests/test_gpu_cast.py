"""GPU parity of the cast / conversion / memory-write kernels through the C ABI: bit-exact against the
CPU oracle, including the reference's LFSR stochastic-rounding stream; the Philox stream is checked
statistically."""
import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util

pytestmark = pytest.mark.gpu

FORMATS = ((abi.BF16, 0, 0), (abi.FP8_143, 7, 2), (abi.FP8_143, 11, 0), (abi.FP8_143, 3, 1), (abi.FP8_152, 15, 0),
           (abi.FP8_152, 20, 2), (abi.FP32, 0, 0))


def accumulators(n, seed=0):
    rng = np.random.default_rng(seed)
    acc = (rng.normal(0, 1, n) * 10.0 ** rng.integers(-9, 9, n)).astype(np.float32)
    acc[:10] = [0, -0.0, np.inf, -np.inf, np.nan, 1e-45, 3e38, -3e38, 448.0, 464.0]
    # the top of each fp8 flavour at bias 7 / 15 (largest finite values, rounding ties, first overflowing values), both signs,
    # scaled to the other biases of FORMATS as well; and a negative NaN
    edges = np.array([240, 247.99, 248, 248.01, 256, 448, 463.99, 464, 464.01, 480, 495.99, 496, 512, 57344, 61439.9, 61440, 65536, 114688, 122880],
                     np.float32)
    tops = np.concatenate([edges * s for s in (1.0, 2.0 ** -4, 2.0 ** 4, 2.0 ** -2, 2.0 ** -5, 2.0 ** -15)])
    acc[10:10 + tops.size] = tops
    acc[10 + tops.size:10 + 2 * tops.size] = -tops
    acc.view(np.uint32)[10 + 2 * tops.size] = 0xFFC00001
    return acc


@pytest.mark.parametrize("od,bias,mode", FORMATS)
def test_activation_bit_exact_all_modes(calc, port, od, bias, mode):
    n = 20011  # not a multiple of the LFSR lane count
    acc = accumulators(n)
    rng = np.random.default_rng(1)
    for rm in (0, 1, 2, 3, 4, 6, 7):
        for relu, clip, ftz, sftz in ((0, 0, 0, 0), (1, 1, 0, 0), (0, 0, 1, 0), (0, 1, 1, 1)):
            cp = abi.make_cast_params(rm, relu, clip_fp=clip, flush_denorms=ftz, stochastic_ftz_fp8=sftz)
            regs = rng.integers(1, 2**32, 256, dtype=np.uint64).astype(np.uint32)
            a1, a2 = acc.copy(), acc.copy()
            o1, o2 = np.zeros(n, abi.NP_DTYPE[od]), np.zeros(n, abi.NP_DTYPE[od])
            rc, regs_after = port.activation(T(o1, od, [n], fp_bias=bias, inf_nan_mode=mode), T(a1, abi.FP32, [n]), cp, regs.copy(), 41)
            assert rc == 0
            calc.set_lfsr(regs, 41)
            calc.do_activation(T(o2, od, [n], fp_bias=bias, inf_nan_mode=mode), T(a2, abi.FP32, [n]), cp)
            assert (o1.view(np.uint8) == o2.view(np.uint8)).all(), (rm, relu, clip, ftz, sftz)
            assert (a1.view(np.uint32) == a2.view(np.uint32)).all()  # ReLU is applied to the accumulator in place
            got, poly = calc.get_lfsr(256)
            assert poly == 41 and (got == regs_after).all()        # registers advance like m_lfsr


def test_lfsr_stream_continues_across_calls(calc, port):
    n1, n2 = 5000, 777
    acc = accumulators(n1 + n2, 3)
    regs = np.arange(2, 258, dtype=np.uint32)
    cp = abi.make_cast_params(abi.RM_SR, clip_fp=True)
    calc.set_lfsr(regs, 37)
    lf = regs.copy()
    for lo, hi in ((0, n1), (n1, n1 + n2)):
        o1, o2 = np.zeros(hi - lo, np.uint16), np.zeros(hi - lo, np.uint16)
        rc, lf = port.activation(T(o1, abi.BF16, [hi - lo]), T(acc[lo:hi].copy(), abi.FP32, [hi - lo]), cp, lf, 37)
        calc.do_activation(T(o2, abi.BF16, [hi - lo]), T(acc[lo:hi].copy(), abi.FP32, [hi - lo]), cp)
        assert (o1 == o2).all()


def test_default_polynomial_and_registers_follow_the_reference_rule(calc):
    # registers i+2; polynomial drawn from mt19937(seed) in [25, 63] (mme_reference_impl.cpp:146-170)
    import intel_gaudi3_software_b200 as pkg
    c = pkg.Calculator(seed=12345)
    regs, poly = c.get_lfsr(256)
    assert (regs == np.arange(2, 258)).all() and 25 <= poly <= 63
    c.close()


def test_philox_stochastic_rounding_is_unbiased(calc):
    """P(round up) must equal the discarded fraction: bin by fraction and compare (5 sigma), and the
    mean of the rounded values must match the mean of the inputs."""
    n = 1 << 20
    rng = np.random.default_rng(5)
    x = rng.uniform(1.0, 2.0, n).astype(np.float32)
    out = np.zeros(n, np.uint16)
    cp = abi.make_cast_params(abi.RM_SR, rng_kind=abi.RNG_PHILOX, rng_seed=99, rng_offset=0)
    calc.do_activation(T(out, abi.BF16, [n]), T(x.copy(), abi.FP32, [n]), cp)
    lo = (x.view(np.uint32) >> 16).astype(np.uint16)
    up = out != lo
    assert ((out == lo) | (out == lo + 1)).all()
    frac = (x.view(np.uint32) & 0xFFFF) / 65536.0
    for b in range(8):
        sel = (frac >= b / 8) & (frac < (b + 1) / 8)
        p_expect, k = frac[sel].mean(), int(sel.sum())
        assert abs(up[sel].mean() - p_expect) < 5 * np.sqrt(p_expect * (1 - p_expect) / k + 1e-12)
    y = util.bf16_to_f32(out).astype(np.float64)
    assert abs(y.mean() - x.astype(np.float64).mean()) < 5 * (2.0 ** -7) / np.sqrt(n)
    # exact values never move, and a different offset gives a different stream
    exact = util.bf16_to_f32(util.f32_to_bf16_rne(x))
    o3 = np.zeros(n, np.uint16)
    calc.do_activation(T(o3, abi.BF16, [n]), T(exact.copy(), abi.FP32, [n]), cp)
    assert (util.bf16_to_f32(o3) == exact).all()
    o4 = np.zeros(n, np.uint16)
    calc.do_activation(T(o4, abi.BF16, [n]), T(x.copy(), abi.FP32, [n]),
                       abi.make_cast_params(abi.RM_SR, rng_kind=abi.RNG_PHILOX, rng_seed=99, rng_offset=4 * n))
    assert (o4 != out).mean() > 0.2


def test_convert_decode_all_codes(calc, port):
    codes = np.tile(np.arange(256, dtype=np.uint8), 5)
    for dt, ew, biases in ((abi.FP8_143, 4, (3, 7, 11, 15)), (abi.FP8_152, 5, (1, 15, 30))):
        for b in biases:
            for mode in (0, 1, 2):
                out = np.zeros(codes.size, np.float32)
                calc.convert(T(out, abi.FP32, [codes.size]), T(codes, dt, [codes.size], fp_bias=b, inf_nan_mode=mode))
                assert (out.view(np.uint32) == port.fp8_to_fp32(codes, ew, b, mode).view(np.uint32)).all()
    h = np.arange(0, 65536, 7, dtype=np.uint32).astype(np.uint16)
    out = np.zeros(h.size, np.float32)
    calc.convert(T(out, abi.FP32, [h.size]), T(h, abi.BF16, [h.size]))
    assert (out.view(np.uint32) == (h.astype(np.uint32) << 16)).all()


def test_convert_encode(calc, port):
    acc = accumulators(30000, 9)
    out = np.zeros(acc.size, np.uint8)
    calc.convert(T(out, abi.FP8_143, [acc.size], fp_bias=7, inf_nan_mode=2), T(acc, abi.FP32, [acc.size]), abi.make_cast_params(abi.RM_NE, clip_fp=True))
    assert (out == port.fp32_to_fp8(acc, 4, 7, abi.RM_NE, None, False, True, False, False, 2)).all()


def test_memory_write(calc, port):
    rng = np.random.default_rng(2)
    n = 50000
    base = rng.normal(0, 1, n).astype(np.float32)
    base[:3] = [1e-40, -1e-40, 3e38]
    src = rng.normal(0, 1, n).astype(np.float32)
    src[2] = 3e38
    base[5:9] = [np.nan, 0.0, -0.0, -1.0]
    src[5:9] = [1.0, -0.0, 0.0, np.nan]
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (0, 1):
                m1, m2 = base.copy(), base.copy()
                assert port.memory_write(T(m1, abi.FP32, [n]), T(src, abi.FP32, [n]), op, rm, clip) == 0
                calc.do_memory_write(T(m2, abi.FP32, [n]), T(src, abi.FP32, [n]), op, rm, clip)
                assert (m1.view(np.uint32) == m2.view(np.uint32)).all(), (op, rm, clip)
    m = base.copy()
    calc.do_memory_write(T(m, abi.FP32, [n]), T(src, abi.FP32, [n]))  # reduction none = copy
    assert (m.view(np.uint32) == src.view(np.uint32)).all()


def test_memory_write_bf16(calc, port):
    from test_numerics_host import bf16_operand_pairs
    a, b = bf16_operand_pairs(np.random.default_rng(31), 100001)
    n = a.size
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (0, 1):
                m1, m2 = a.copy(), a.copy()
                assert port.memory_write(T(m1, abi.BF16, [n]), T(b.copy(), abi.BF16, [n]), op, rm, clip) == 0
                calc.do_memory_write(T(m2, abi.BF16, [n]), T(b.copy(), abi.BF16, [n]), op, rm, clip)
                assert (m1 == m2).all(), (op, rm, clip, int((m1 != m2).sum()))
    with pytest.raises(Exception, match="not implemented"):   # the reference rejects fp8_143 reductions too
        x = np.zeros(16, np.uint8)
        calc.do_memory_write(T(x, abi.FP8_143, [16], fp_bias=7), T(x.copy(), abi.FP8_143, [16], fp_bias=7), abi.RED_ADD, 0)


def test_memory_write_fp8_152_every_operand_pair(calc, port):
    """All 256 x 256 pairs of codes (twice over, plus a ragged tail, so the vector path and the scalar tail both run), every
    reduction, direction and clip flag, bit for bit against the oracle."""
    a = np.concatenate([np.repeat(np.arange(256, dtype=np.uint8), 256)] * 2 + [np.arange(7, dtype=np.uint8)])
    b = np.concatenate([np.tile(np.arange(256, dtype=np.uint8), 256)] * 2 + [np.arange(7, dtype=np.uint8)[::-1]])
    n = a.size
    kw = dict(fp_bias=15, inf_nan_mode=abi.INFNAN_FULL)
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (0, 1):
                m1, m2 = a.copy(), a.copy()
                assert port.memory_write(T(m1, abi.FP8_152, [n], **kw), T(b.copy(), abi.FP8_152, [n], **kw), op, rm, clip) == 0
                calc.do_memory_write(T(m2, abi.FP8_152, [n], **kw), T(b.copy(), abi.FP8_152, [n], **kw), op, rm, clip)
                assert (m1 == m2).all(), (op, rm, clip, int((m1 != m2).sum()))


def test_dma_transpose_and_copy(calc):
    rng = np.random.default_rng(4)
    a = rng.integers(0, 65536, 37 * 53 * 3).astype(np.uint16)
    out = np.zeros_like(a)
    calc.do_dma(T(out, abi.BF16, [53, 37, 3]), T(a, abi.BF16, [37, 53, 3]), abi.OP_TRANS)
    assert (out.reshape(3, 37, 53) == a.reshape(3, 53, 37).transpose(0, 2, 1)).all()
    out2 = np.zeros_like(a)
    calc.do_dma(T(out2, abi.BF16, [37, 53, 3]), T(a, abi.BF16, [37, 53, 3]), abi.OP_MEMCPY)
    assert (out2 == a).all()
