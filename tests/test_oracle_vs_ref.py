"""Checks the C restatement against the compiled, unmodified reference on fresh random inputs
(wider than the committed golden vectors). Skipped where oracle/_ref is not built."""
import itertools

import numpy as np

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util


def same(a, b):
    return (a.view(np.uint32) == b.view(np.uint32)).all()


def test_decode_all_codes(port, ref):
    codes = np.arange(256, dtype=np.uint8)
    for ew, biases in ((4, (3, 7, 11, 15)), (5, tuple(range(1, 31)))):
        for b in biases:
            for mode in (0, 1, 2):
                assert same(port.fp8_to_fp32(codes, ew, b, mode), ref.fp8_to_fp32(codes, ew, b, mode))


def test_casts_random(port, ref):
    rng = np.random.default_rng(3)
    n = 60000
    bits = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    ex = rng.integers(127 - 40, 127 + 20, size=n).astype(np.uint32)
    b2 = (bits & 0x807FFFFF) | (ex << 23)
    allbits = np.concatenate([bits, b2, b2 & 0xFFF00000, b2 & 0xFFF80000])
    lfsr = rng.integers(0, 2**32, size=allbits.size, dtype=np.uint64).astype(np.uint32)
    lfsr[:500] = 0
    for rm in (0, 1, 2, 3, 4, 6, 7):
        for clip, ftz, cii in itertools.product((0, 1), (0, 1), (0, 1)):
            assert (port.fp32_to_bf16(allbits, rm, lfsr, clip, ftz, cii) == ref.fp32_to_bf16(allbits, rm, lfsr, clip, ftz, cii)).all()
        for ew, b, mode in ((4, 3, 0), (4, 7, 2), (4, 11, 1), (4, 15, 2), (5, 1, 0), (5, 15, 0), (5, 30, 2)):
            for ftz, clip, cii, sftz in ((0, 0, 0, 0), (1, 0, 0, 0), (0, 1, 1, 0), (1, 1, 0, 1), (0, 0, 0, 1)):
                a = port.fp32_to_fp8(allbits, ew, b, rm, lfsr, ftz, clip, cii, sftz, mode)
                c = ref.fp32_to_fp8(allbits, ew, b, rm, lfsr, ftz, clip, cii, sftz, mode)
                assert (a == c).all(), (ew, b, mode, rm, ftz, clip, cii, sftz)


def test_dot_products(port, ref):
    rng = np.random.default_rng(4)
    for n in (1, 5, 8, 9, 64, 1000, 4096):
        for trial in range(6):
            a, b = util.gen_bf16(rng, n), util.gen_bf16(rng, n)
            if trial % 3 == 2:
                a = util.f32_to_bf16_rne((rng.normal(0, 1, n) * 10.0 ** rng.integers(-18, 18, n)).astype(np.float32))
            x = np.float32(port.fma_vec(abi.BF16, abi.BF16, a, b))
            y = np.float32(ref.fma_vec(abi.BF16, abi.BF16, a, b))
            assert x.view(np.uint32) == y.view(np.uint32)
        for ta, tb in ((9, 9), (10, 9), (9, 10), (10, 10)):
            for mode in (0, 1, 2):
                a = rng.integers(0, 256, n).astype(np.uint8)
                b = rng.integers(0, 256, n).astype(np.uint8)
                kw = dict(bias_a=7 if ta == 9 else 15, bias_b=11 if tb == 9 else 15, mode_a=mode, mode_b=mode)
                x = np.float32(port.fma_vec(ta, tb, a, b, **kw))
                y = np.float32(ref.fma_vec(ta, tb, a, b, **kw))
                assert x.view(np.uint32) == y.view(np.uint32)


def test_bgemm_strided_broadcast(port, ref):
    rng = np.random.default_rng(5)
    for op in (abi.OP_AB, abi.OP_ABT, abi.OP_ATB, abi.OP_ATBT):
        M, N, K = 13, 10, 21
        xs = [K, M] if op in (abi.OP_AB, abi.OP_ABT) else [M, K]
        ws = [N, K] if op in (abi.OP_AB, abi.OP_ATB) else [K, N]
        xsz, wsz, osz = xs + [3, 1, 2], ws + [1, 2, 2], [N, M, 3, 2, 2]
        xstr = [1, xs[0] + 3]
        xstr += [xstr[1] * xs[1]]
        xstr += [xstr[2] * 3]
        xstr += [xstr[3]]
        xbuf = util.gen_bf16(rng, xstr[4] * 2)
        wbuf = util.gen_bf16(rng, int(np.prod(wsz)))
        ostr = [1, N + 2, (N + 2) * M, (N + 2) * M * 3, (N + 2) * M * 6]
        o1 = np.full(ostr[4] * 2, 7.0, np.float32)
        o2 = o1.copy()
        x, w = T(xbuf, abi.BF16, xsz, xstr), T(wbuf, abi.BF16, wsz)
        assert port.bgemm(T(o1, abi.FP32, osz, ostr), x, w, op) == 0
        assert ref.bgemm(T(o2, abi.FP32, osz, ostr), x, w, op) == 0
        assert same(o1, o2), op


def test_conv_3d(port, ref):
    rng = np.random.default_rng(6)
    cp = abi.make_conv_params(3, (1, 1, 1), (1, 1, 1), (1, 1, 1))
    xs, ws, ys = [4, 5, 5, 4, 2], [3, 4, 2, 2, 2], [3, 6, 6, 5, 2]
    xb, wb, yb = util.gen_bf16(rng, int(np.prod(xs)), "normal"), util.gen_bf16(rng, int(np.prod(ws)), "normal", 0.1), util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.01)
    x, w, y = T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), T(yb, abi.BF16, ys)
    for op, shp in ((abi.OP_FWD, ys), (abi.OP_DEDX, xs), (abi.OP_DEDW, ws)):
        o1 = np.full(int(np.prod(shp)), 3.0, np.float32)
        o2 = o1.copy()
        assert port.conv(T(o1, abi.FP32, shp), x, w, y, cp, op) == 0
        assert ref.conv(T(o2, abi.FP32, shp), x, w, y, cp, op) == 0
        assert same(o1, o2), op


def test_memory_write_reductions(port, ref):
    rng = np.random.default_rng(7)
    m1 = rng.normal(0, 1, 300).astype(np.float32)
    m1[:3] = [1e-40, -1e-40, 3e38]
    m2 = m1.copy()
    s = rng.normal(0, 1, 300).astype(np.float32)
    s[2] = 3e38
    m1[5:9] = [np.nan, 0.0, -0.0, -1.0]
    s[5:9] = [1.0, -0.0, 0.0, np.nan]
    m2 = m1.copy()
    base = m1.copy()
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (0, 1):
                m1[:], m2[:] = base, base
                assert port.memory_write(T(m1, abi.FP32, [300]), T(s, abi.FP32, [300]), op, rm, clip) == 0
                assert ref.memory_write(T(m2, abi.FP32, [300]), T(s, abi.FP32, [300]), op, rm, clip) == 0
                assert same(m1, m2), (op, rm, clip)


def test_memory_write_fp8_152_reductions_on_every_operand_pair(port, ref):
    a = np.repeat(np.arange(256, dtype=np.uint8), 256)
    b = np.tile(np.arange(256, dtype=np.uint8), 256)
    n = a.size
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (False, True):
                if op in (abi.RED_MIN, abi.RED_MAX) and (rm or clip):
                    continue
                m1, m2 = a.copy(), a.copy()
                assert port.memory_write(T(m1, abi.FP8_152, [n], fp_bias=15), T(b.copy(), abi.FP8_152, [n], fp_bias=15), op, rm, clip) == 0
                assert ref.memory_write(T(m2, abi.FP8_152, [n], fp_bias=15), T(b.copy(), abi.FP8_152, [n], fp_bias=15), op, rm, clip) == 0
                bad = np.nonzero(m1 != m2)[0]
                assert bad.size == 0, (op, rm, clip, bad.size, [(hex(a[i]), hex(b[i]), hex(m1[i]), hex(m2[i])) for i in bad[:8]])


def test_memory_write_bf16_reductions(port, ref):
    from test_numerics_host import bf16_operand_pairs
    a, b = bf16_operand_pairs(np.random.default_rng(29), 120000)
    n = a.size
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (False, True):
                m1, m2 = a.copy(), a.copy()
                assert port.memory_write(T(m1, abi.BF16, [n]), T(b.copy(), abi.BF16, [n]), op, rm, clip) == 0
                assert ref.memory_write(T(m2, abi.BF16, [n]), T(b.copy(), abi.BF16, [n]), op, rm, clip) == 0
                assert (m1 == m2).all(), (op, rm, clip, int((m1 != m2).sum()))
