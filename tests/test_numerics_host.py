"""The product's conversion functions (csrc/numerics.cuh) compiled for the host and compared, bit for
bit, with the CPU oracle. This checks the device code's arithmetic on a machine without a GPU; the
GPU tests repeat the comparison through the kernels."""
import ctypes as C
import os
import subprocess

import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SRC = os.path.join(ROOT, "tests", "hostcheck", "numerics_host.cpp")
SO = os.path.join(ROOT, "tests", "hostcheck", "libnumerics_host.so")


@pytest.fixture(scope="module")
def hc():
    inc = os.path.join(ROOT, "intel_gaudi3_software_b200", "csrc")
    newest = max(os.path.getmtime(f) for f in [SRC] + [os.path.join(inc, h) for h in ("numerics.cuh", "schedule.cuh", "gaudi3_exact.cuh")])
    if not os.path.exists(SO) or os.path.getmtime(SO) < newest:
        subprocess.check_call(["g++", "-std=c++17", "-O2", "-fPIC", "-shared", "-I" + inc, "-o", SO, SRC])
    return C.CDLL(SO)


def inputs():
    rng = np.random.default_rng(11)
    n = 40000
    bits = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    ex = rng.integers(127 - 40, 127 + 20, size=n).astype(np.uint32)
    b2 = (bits & 0x807FFFFF) | (ex << 23)
    special = np.array([0, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 1, 0x80000001, 0x007FFFFF,
                        0x7F7FFFFF, 0xFF7FFFFF], dtype=np.uint32)
    allbits = np.concatenate([bits, b2, b2 & 0xFFF00000, b2 & 0xFFF80000, special])
    lfsr = rng.integers(0, 2**32, size=allbits.size, dtype=np.uint64).astype(np.uint32)
    lfsr[:300] = 0
    return allbits, lfsr


def test_decode(hc, port):
    codes = np.arange(256, dtype=np.uint8)
    out = np.zeros(256, np.uint32)
    for ew, biases in ((4, (3, 7, 11, 15)), (5, (1, 15, 30))):
        for b in biases:
            for mode in (0, 1, 2):
                hc.hc_fp8_decode(codes.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_size_t(256), ew, b, mode)
                assert (out == port.fp8_to_fp32(codes, ew, b, mode).view(np.uint32)).all()


def test_casts(hc, port):
    bits, lfsr = inputs()
    n = bits.size

    def run(out_dtype, ew, bias, mode, rm, relu, clip, cii, ftz, sftz):
        out = np.zeros(n * abi.ELEM_SIZE[out_dtype], np.uint8)
        hc.hc_cast(bits.ctypes.data_as(C.c_void_p), out.ctypes.data_as(C.c_void_p), C.c_size_t(n), out_dtype, ew, bias, mode, rm,
                   relu, clip, cii, ftz, sftz, lfsr.ctypes.data_as(C.c_void_p))
        return out
    for rm in (0, 1, 2, 3, 4, 6, 7):
        for clip, ftz, cii in ((0, 0, 0), (1, 0, 0), (1, 1, 1), (0, 1, 0)):
            got = run(abi.BF16, 0, 0, 0, rm, 0, clip, cii, ftz, 0).view(np.uint16)
            assert (got == port.fp32_to_bf16(bits, rm, lfsr, clip, ftz, cii)).all(), (rm, clip, ftz, cii)
        for dt, ew, b, mode in ((abi.FP8_143, 4, 3, 0), (abi.FP8_143, 4, 7, 2), (abi.FP8_143, 4, 11, 1), (abi.FP8_152, 5, 15, 0), (abi.FP8_152, 5, 30, 2)):
            for ftz, clip, cii, sftz in ((0, 0, 0, 0), (1, 0, 0, 0), (0, 1, 1, 0), (1, 1, 0, 1), (0, 0, 0, 1)):
                got = run(dt, ew, b, mode, rm, 0, clip, cii, ftz, sftz)
                assert (got == port.fp32_to_fp8(bits, ew, b, rm, lfsr, ftz, clip, cii, sftz, mode)).all(), (dt, b, mode, rm, ftz, clip, cii, sftz)


def test_epilogue_flat_casts_equal_the_general_ones(hc):
    """The straight-line casts of the GEMM epilogue return the bits of the general casts on every input: every binade and its
    edges, zeros, infinities, NaN, every rounding mode, Inf/NaN convention and clip flag (fp8: without the flush flags)."""
    bits, lfsr = inputs()
    rng = np.random.default_rng(12)
    # every exponent with random mantissas, and the neighbourhood of every power of two, so that each binade boundary of
    # each fp8 flavour is hit
    ex = np.repeat(np.arange(256, dtype=np.uint32), 64)
    dense = (rng.integers(0, 2**23, ex.size).astype(np.uint32) | (ex << 23))
    edges = np.concatenate([(ex << 23) + d for d in (0, 1, 0x7FFFFF, 0x400000, 0x3FFFFF, 0x400001, 0x100000, 0x080000, 0x0FFFFF)]).astype(np.uint32)
    bits = np.concatenate([bits, dense, dense | 0x80000000, edges, edges | 0x80000000])
    lfsr = np.concatenate([lfsr, rng.integers(0, 2**32, bits.size - lfsr.size, dtype=np.uint64).astype(np.uint32)])
    lfsr[-2000:] = 0
    n = bits.size
    slow = np.zeros(n, np.uint8)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731

    def both(out_dtype, ew, bias, mode, rm, clip, cii, ftz):
        es = abi.ELEM_SIZE[out_dtype]
        a, b = np.zeros(n * es, np.uint8), np.zeros(n * es, np.uint8)
        hc.hc_cast(vp(bits), vp(a), C.c_size_t(n), out_dtype, ew, bias, mode, rm, 0, clip, cii, ftz, 0, vp(lfsr))
        assert hc.hc_cast_flat(vp(bits), vp(b), vp(slow), C.c_size_t(n), out_dtype, ew, bias, mode, rm, clip, cii, ftz, vp(lfsr)) == 0
        return a, b
    for rm in (0, 1, 2, 3, 4, 6, 7):
        for clip, ftz, cii in ((0, 0, 0), (1, 0, 0), (1, 1, 1), (0, 1, 0), (1, 0, 1)):
            a, b = both(abi.BF16, 0, 0, 0, rm, clip, cii, ftz)
            assert (a == b).all(), (rm, clip, ftz, cii)
        for dt, ew, biases in ((abi.FP8_143, 4, (1, 3, 7, 11, 15)), (abi.FP8_152, 5, (1, 15, 30, 31))):
            for bias in biases:
                for mode in (0, 1, 2):
                    for clip, cii in ((0, 0), (1, 0), (1, 1)):
                        a, b = both(dt, ew, bias, mode, rm, clip, cii, 0)
                        assert (a == b).all(), (dt, bias, mode, rm, clip, cii, [hex(v) for v in bits[a != b][:5]], a[a != b][:5], b[a != b][:5])


def test_hardware_fp8_path_constants(hc):
    """The rescale, overflow thresholds and constant codes around the hardware fp8 conversion give the general cast's bits for
    every 1-4-3 convention and the IEEE-like 1-5-2, every bias and clip flag (the hardware conversion itself is modelled on
    the host as a saturating nearest-even cast into the hardware format; the GPU tests run the real instruction)."""
    rng = np.random.default_rng(13)
    ex = np.repeat(np.arange(256, dtype=np.uint32), 96)
    dense = rng.integers(0, 2**23, ex.size).astype(np.uint32) | (ex << 23)
    edges = np.concatenate([(ex << 23) + d for d in (0, 1, 0x7FFFFF, 0x400000, 0x3FFFFF, 0x400001, 0x100000, 0x080000, 0x0FFFFF, 0x700000, 0x780000,
                                                      0x680000, 0x6FFFFF, 0x680001, 0x500000, 0x4FFFFF, 0x500001)]).astype(np.uint32)
    special = np.array([0, 0x7F800000, 0x7FC00000, 0x7F800001, 0x7FFFFFFF], np.uint32)
    bits = np.concatenate([dense, edges, special])
    bits = np.concatenate([bits, bits | 0x80000000])
    n = bits.size
    zeros = np.zeros(n, np.uint32)
    vp = lambda a: a.ctypes.data_as(C.c_void_p)  # noqa: E731
    for dt, ew, biases, modes in ((abi.FP8_143, 4, (1, 3, 7, 11, 15), (0, 1, 2)), (abi.FP8_152, 5, (1, 15, 24, 31), (0,))):
        for bias in biases:
            for mode in modes:
                for clip, cii in ((0, 0), (1, 0), (1, 1), (0, 1)):
                    want, got = np.zeros(n, np.uint8), np.zeros(n, np.uint8)
                    hc.hc_cast(vp(bits), vp(want), C.c_size_t(n), dt, ew, bias, mode, 0, 0, clip, cii, 0, 0, vp(zeros))
                    assert hc.hc_cast_fp8_hw_model(vp(bits), vp(got), C.c_size_t(n), dt, ew, bias, mode, clip, cii) == 0
                    bad = np.flatnonzero(want != got)
                    assert bad.size == 0, (dt, bias, mode, clip, cii, [(hex(bits[i]), hex(want[i]), hex(got[i])) for i in bad[:6]])
    # the conventions the hardware 1-5-2 format cannot express are not routed there
    assert hc.hc_cast_fp8_hw_model(vp(bits), vp(got), C.c_size_t(n), abi.FP8_152, 5, 15, 2, 0, 0) == -1


def test_foreign_code_predicate(hc, port):
    """A code is 'foreign' exactly when the reference decode differs from the tensor cores' decode
    (OCP E4M3 = the 1-4-3 'minimal' convention at bias 7; OCP E5M2 = the 1-5-2 'full' convention at bias 15)."""
    codes = np.arange(256, dtype=np.uint8)
    for ew, hw_bias, hw_mode in ((4, 7, 2), (5, 15, 0)):
        hw = port.fp8_to_fp32(codes, ew, hw_bias, hw_mode).view(np.uint32)
        for mode in (0, 1, 2):
            mine = port.fp8_to_fp32(codes, ew, hw_bias, mode).view(np.uint32)
            for c in range(256):
                assert bool(hc.hc_fp8_foreign(c, ew, mode)) == bool(hw[c] != mine[c]), (ew, mode, c)


def test_lfsr_step(hc, port):
    hc.hc_lfsr.restype = C.c_uint32
    v = 0xDEADBEEF
    for _ in range(200):
        nxt = hc.hc_lfsr(C.c_uint32(v), C.c_uint32(37))
        assert nxt == port.lfsr32(v, 37)
        v = nxt


def test_philox_known_answers(hc):
    """Philox4x32-10 known-answer vectors of the Random123 distribution (kat_vectors)."""
    def block(ctr, key):
        c = (C.c_uint32 * 4)(*ctr)
        hc.hc_philox_block(c, C.c_uint32(key[0]), C.c_uint32(key[1]))
        return list(c)
    assert block([0, 0, 0, 0], [0, 0]) == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]
    assert block([0xFFFFFFFF] * 4, [0xFFFFFFFF, 0xFFFFFFFF]) == [0x408F276D, 0x41C83B0E, 0xA20BC7C6, 0x6D5451FD]
    assert block([0x243F6A88, 0x85A308D3, 0x13198A2E, 0x03707344], [0xA4093822, 0x299F31D0]) == [0xD16CFE09, 0x94FDCCEB, 0x5001E420, 0x24126EA1]


def test_philox_half_stream_for_16_bit_outputs(hc):
    """bf16 casts draw 16 random bits per element, eight elements per Philox block: the per-element, per-four and per-eight
    forms agree, the words are (h << 16) | 0x8000 with h uniform, and a different stream from the 32-bit one."""
    hc.hc_philox_half.restype = C.c_uint32
    hc.hc_philox.restype = C.c_uint32
    w8, w4a, w4b = (np.zeros(8, np.uint32), np.zeros(4, np.uint32), np.zeros(4, np.uint32))
    for base in (0, 8, 4096):
        hc.hc_philox_halves(C.c_uint64(9), C.c_uint64(16), C.c_uint64(base), w8.ctypes.data_as(C.c_void_p), w4a.ctypes.data_as(C.c_void_p),
                            w4b.ctypes.data_as(C.c_void_p))
        single = np.array([hc.hc_philox_half(C.c_uint64(9), C.c_uint64(16), C.c_uint64(base + i)) for i in range(8)], dtype=np.uint32)
        assert (w8 == single).all() and (np.concatenate([w4a, w4b]) == single).all()
        assert (hc.hc_philox_half(C.c_uint64(9), C.c_uint64(0), C.c_uint64(base + 16)) == single[0])   # offset and index add up
    w = np.array([hc.hc_philox_half(C.c_uint64(5), C.c_uint64(0), C.c_uint64(i)) for i in range(40000)], dtype=np.uint64)
    assert ((w & 0xFFFF) == 0x8000).all()
    h = (w >> 16).astype(np.float64)
    assert abs(h.mean() / 65536 - 0.5) < 0.01 and len(np.unique(h)) > 15000
    w32 = np.array([hc.hc_philox(C.c_uint64(5), C.c_uint64(0), C.c_uint64(i)) for i in range(64)], dtype=np.uint64)
    assert ((w32 >> 16) != (w[:64] >> 16)).mean() > 0.9


def sr_inputs(discard_bits, e_small, e_top):
    """fp32 values in groups of eight with a raw Philox-like block each: every exponent and sign, mantissas with structured
    and random low parts, and random halves placed at, just below and just above the value's own discarded bits (the
    decision's change point), besides uniform ones. Some groups hold a value near the top of the range, Inf or NaN."""
    rng = np.random.default_rng(23)
    n = 1 << 21
    sign = rng.integers(0, 2, n, dtype=np.uint64) << 31
    ex = rng.integers(0, 256, n, dtype=np.uint64)
    where = rng.integers(0, 4, n)
    ex = np.where(where == 0, rng.integers(e_small - 9, e_small + 3, n).astype(np.uint64), ex)   # the output's subnormal range and below
    ex = np.where(where == 1, rng.integers(e_top - 2, e_top + 2, n).astype(np.uint64), ex)       # its largest binade and the overflow
    ex = np.clip(ex, 0, 255).astype(np.uint64) << 23
    man = rng.integers(0, 1 << 23, n, dtype=np.uint64)
    kind = rng.integers(0, 6, n)
    man = np.where(kind == 0, man & ~np.uint64((1 << discard_bits) - 1), man)          # exactly representable
    man = np.where(kind == 1, man | np.uint64((1 << discard_bits) - 1), man)           # all discarded bits set
    man = np.where(kind == 2, (man & ~np.uint64((1 << discard_bits) - 1)) | np.uint64(1), man)
    bits = (sign | ex | man).astype(np.uint32)
    special = np.array([0, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 0x7FFFFFFF, 0xFFFFFFFF, 1, 0x007FFFFF, 0x7F7FFFFF,
                        0xFF7FFFFF, 0x7F7F0000, 0x7F7F0001, 0x7F7EFFFF], dtype=np.uint32)
    bits[: special.size * 8 : 8] = special                                             # one special value in each of the first groups
    disc = (bits.astype(np.uint64) & np.uint64((1 << discard_bits) - 1)) >> np.uint64(discard_bits - 16)   # top 16 discarded bits (normal result)
    pick = rng.integers(0, 5, n)
    h = rng.integers(0, 1 << 16, n, dtype=np.uint64)
    h = np.where(pick == 0, disc, h)
    h = np.where(pick == 1, (disc - 1) & 0xFFFF, h)
    h = np.where(pick == 2, (disc + 1) & 0xFFFF, h)
    h = np.where(rng.integers(0, 64, n) == 0, np.uint64(0), h)
    h = np.where(rng.integers(0, 64, n) == 0, np.uint64(0xFFFF), h)
    blocks = (h[0::2] | (h[1::2] << 16)).astype(np.uint32)                             # element 2j: low half of word j
    return bits, np.ascontiguousarray(blocks)


def test_stochastic_rounding_as_an_addition_equals_the_straight_line_cast(hc):
    """sr_bf16_group8 / sr_fp8_group8 (one integer addition per element, the straight-line cast for groups near the top of
    the range) against f32_to_bf16_flat<RM_SR> / f32_to_fp8_flat<RM_SR> with the same random halves."""
    vp = lambda a: a.ctypes.data_as(C.c_void_p)
    cases = [(abi.BF16, 0, 0, 0, 16)]   # (type, exponent width, bias, Inf/NaN convention, bits a normal result discards)
    for ew, dt, biases, modes in ((4, abi.FP8_143, (3, 7, 11, 15), (0, 1, 2)), (5, abi.FP8_152, (15, 1, 24), (0, 2))):
        cases += [(dt, ew, b, m, 23 - (7 - ew)) for b in biases for m in modes]
    for dt, ew, bias, mode, discard in cases:
        e_small = 128 - bias if ew else 1
        e_top = (127 - bias + (1 << ew) - (1 if mode == 0 else 0)) if ew else 254
        bits, blocks = sr_inputs(discard, e_small, e_top)
        es = 2 if dt == abi.BF16 else 1
        for clip, cii, canon in ((0, 0, 0), (1, 0, 1), (1, 1, 0)):
            fast, flat = np.zeros(bits.size * es, np.uint8), np.zeros(bits.size * es, np.uint8)
            hc.hc_sr_groups(vp(bits), vp(blocks), C.c_size_t(bits.size // 8), dt, ew, bias, mode, clip, cii, canon, vp(fast), vp(flat))
            bad = np.nonzero(fast != flat)[0]
            assert bad.size == 0, (dt, ew, bias, mode, clip, cii, hex(int(bits[bad[0] // es])), int(fast[bad[0]]), int(flat[bad[0]]))
        # the two roundings must both occur (the change points are inside the sample)
        assert len(np.unique(flat)) > (200 if es == 1 else 250)
    c4, w8 = np.zeros(4, np.uint32), np.zeros(8, np.uint32)
    hc.hc_philox_half.restype = C.c_uint32
    hc.hc_philox_block8(C.c_uint64(9), C.c_uint64(16), C.c_uint64(4096), vp(c4), vp(w8))
    assert [hc.hc_philox_half(C.c_uint64(9), C.c_uint64(16), C.c_uint64(4096 + i)) for i in range(8)] == w8.tolist()


def test_philox_word_never_zero_and_uniform(hc):
    hc.hc_philox.restype = C.c_uint32
    w = np.array([hc.hc_philox(C.c_uint64(5), C.c_uint64(0), C.c_uint64(i)) for i in range(20000)], dtype=np.uint64)
    assert (w != 0).all()
    # top bit and a middle bit are fair coins (5 sigma)
    for bit in (31, 13):
        ones = int(((w >> bit) & 1).sum())
        assert abs(ones - 10000) < 5 * 71


def comparator_pairs(dtype, rng, n=6000):
    """Pairs that land on every branch of the rule: identical, a few ulps apart, far apart, sign flips, zeros, Inf / NaN."""
    if dtype == abi.FP32:
        a = (rng.normal(0, 1, n) * 10.0 ** rng.integers(-3, 4, n)).astype(np.float32)
        b = a.copy()
        k = n // 6
        b[:k] = (a[:k].view(np.uint32) + rng.integers(0, 12, k).astype(np.uint32)).view(np.float32)
        b[k:2 * k] = a[k:2 * k] * rng.uniform(0.8, 1.2, k).astype(np.float32)
        b[2 * k:3 * k] = -a[2 * k:3 * k]
        b[3 * k:3 * k + 8] = [0, -0.0, np.inf, -np.inf, np.nan, 1e-3, 0.04, 0.06]
        a[3 * k + 4:3 * k + 8] = [1.0, 0.0, 0.0, 0.0]
        return a.view(np.uint32), b.view(np.uint32)
    if dtype == abi.BF16:
        a = rng.integers(0, 65536, n).astype(np.uint16)
        b = a.copy()
        k = n // 4
        b[:k] = (a[:k].astype(np.int32) + rng.integers(-9, 10, k)).astype(np.uint16)
        b[k:2 * k] = rng.integers(0, 65536, k).astype(np.uint16)
        b[2 * k:3 * k] = a[2 * k:3 * k] ^ 0x8000
        return a, b
    a = rng.integers(0, 256, n).astype(np.uint8)
    b = a.copy()
    k = n // 4
    b[:k] = (a[:k].astype(np.int32) + rng.integers(-6, 7, k)).astype(np.uint8)
    b[k:2 * k] = rng.integers(0, 256, k).astype(np.uint8)
    b[2 * k:3 * k] = a[2 * k:3 * k] ^ 0x80
    return a, b


def test_comparator_rule_matches_reference(hc, ref):
    rng = np.random.default_rng(17)
    for dtype, bias, mode in ((abi.FP32, 0, 0), (abi.BF16, 0, 0), (abi.FP8_143, 7, 2), (abi.FP8_143, 3, 0), (abi.FP8_143, 15, 1),
                              (abi.FP8_152, 15, 0), (abi.FP8_152, 24, 2)):
        for cd in (1, 64, 2304, 200704):
            a, b = comparator_pairs(dtype, rng)
            mine = np.zeros(a.size, np.uint8)
            hc.hc_compare(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), mine.ctypes.data_as(C.c_void_p), C.c_size_t(a.size),
                          dtype, bias, mode, cd)
            want = ref.compare_elements(dtype, bias, mode, cd, a, b)
            assert (mine == want).all(), (dtype, bias, mode, cd, np.nonzero(mine != want)[0][:5])


def bf16_operand_pairs(rng, n=300000):
    """Random bit patterns, near-cancelling pairs, operands many binades apart, and every special value."""
    a = rng.integers(0, 65536, n).astype(np.uint16)
    b = rng.integers(0, 65536, n).astype(np.uint16)
    k = n // 4
    b[:k] = (a[:k] ^ 0x8000) + rng.integers(-3, 4, k).astype(np.uint16)                  # a - (a +- few ulps)
    near = rng.integers(-12, 13, k)
    b[k:2 * k] = ((a[k:2 * k].astype(np.int32) + near * 128) & 0xFFFF).astype(np.uint16)   # exponents within 12 binades
    b[2 * k:2 * k + k // 2] = a[2 * k:2 * k + k // 2]                                        # doubling
    special = np.array([0, 0x8000, 0x0001, 0x8001, 0x007F, 0x0080, 0x8080, 0x0081, 0x7F7F, 0xFF7F, 0x7F80, 0xFF80, 0x7FC0, 0xFFFF, 0x3F80,
                        0xBF80, 0x7F00, 0xFF00, 0x0100, 0x8100], np.uint16)
    sa, sb = np.meshgrid(special, special)
    return np.concatenate([a, sa.reshape(-1)]), np.concatenate([b, sb.reshape(-1)])


def test_bf16_memory_write_matches_reference(hc, ref):
    rng = np.random.default_rng(23)
    a, b = bf16_operand_pairs(rng)
    n = a.size
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (False, True):
                if op in (abi.RED_MIN, abi.RED_MAX) and (rm or clip):
                    continue
                want = a.copy()
                assert ref.memory_write(T(want, abi.BF16, [n]), T(b.copy(), abi.BF16, [n]), op, rm, clip) == 0
                mine = a.copy()
                hc.hc_bf16_rmw(mine.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), C.c_size_t(n), op, rm, int(clip))
                bad = np.nonzero(mine != want)[0]
                assert bad.size == 0, (op, rm, clip, bad.size, [(hex(a[i]), hex(b[i]), hex(mine[i]), hex(want[i])) for i in bad[:6]])


def test_fp8_152_memory_write_matches_reference_on_every_operand_pair(hc, ref):
    """All 256 x 256 pairs of fp8_152 codes through every reduction, direction and clip flag: the product's arithmetic
    (fp8_152_rmw) against doMemoryWrite of the compiled reference, bit for bit."""
    a = np.repeat(np.arange(256, dtype=np.uint8), 256)
    b = np.tile(np.arange(256, dtype=np.uint8), 256)
    n = a.size
    for op in (abi.RED_ADD, abi.RED_SUB, abi.RED_MIN, abi.RED_MAX, abi.RED_MAX_0):
        for rm in (0, 1, 2, 3):
            for clip in (False, True):
                if op in (abi.RED_MIN, abi.RED_MAX) and (rm or clip):
                    continue
                want = a.copy()
                assert ref.memory_write(T(want, abi.FP8_152, [n], fp_bias=15), T(b.copy(), abi.FP8_152, [n], fp_bias=15), op, rm, clip) == 0
                mine = a.copy()
                hc.hc_fp8_152_rmw(mine.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), C.c_size_t(n), op, rm, int(clip))
                bad = np.nonzero(mine != want)[0]
                assert bad.size == 0, (op, rm, clip, bad.size, [(hex(a[i]), hex(b[i]), hex(mine[i]), hex(want[i])) for i in bad[:8]])


def test_gaudi3_tree_restatement_matches_reference(hc, ref):
    """g3_tree8 (the block step of the bit-exact GPU mode) against fma_vec of the compiled reference: bf16 and fp8 vectors of
    many lengths, wide exponent spreads, cancellation, denormals, Inf and NaN."""
    rng = np.random.default_rng(41)
    hc.hc_g3_dot.restype = C.c_uint32
    cases = 0
    for n in (1, 7, 8, 9, 64, 200, 1031):
        for kind in range(6):
            if kind < 3:   # bf16
                a = rng.integers(0, 65536, n).astype(np.uint16)
                b = rng.integers(0, 65536, n).astype(np.uint16)
                if kind == 1:    # moderate exponents: sums that cancel
                    a = (a & 0x807F) | (rng.integers(120, 134, n).astype(np.uint16) << 7)
                    b = (b & 0x807F) | (rng.integers(120, 134, n).astype(np.uint16) << 7)
                if kind == 2:    # no Inf / NaN, denormals included
                    a[(a & 0x7F80) == 0x7F80] = 0x0001
                    b[(b & 0x7F80) == 0x7F80] = 0x8001
                want = np.float32(ref.fma_vec(abi.BF16, abi.BF16, a, b)).view(np.uint32)
                fa, fb = a.astype(np.uint32) << 16, b.astype(np.uint32) << 16
            else:          # fp8, mixed formats, biases and modes
                ta, tb = ((abi.FP8_143, abi.FP8_143), (abi.FP8_152, abi.FP8_143), (abi.FP8_152, abi.FP8_152))[kind - 3]
                ba, bb = (7, 11) if kind == 3 else (15, 3) if kind == 4 else (20, 15)
                ma, mb = (2, 0) if kind == 3 else (0, 1) if kind == 4 else (1, 2)
                a = rng.integers(0, 256, n).astype(np.uint8)
                b = rng.integers(0, 256, n).astype(np.uint8)
                want = np.float32(ref.fma_vec(ta, tb, a, b, ba, bb, ma, mb)).view(np.uint32)
                fa = ref.fp8_to_fp32(a, 4 if ta == abi.FP8_143 else 5, ba, ma)
                fb = ref.fp8_to_fp32(b, 4 if tb == abi.FP8_143 else 5, bb, mb)
            fa, fb = (np.ascontiguousarray(v).view(np.uint32) if np.asarray(v).dtype == np.float32 else np.ascontiguousarray(v, np.uint32) for v in (fa, fb))
            got = hc.hc_g3_dot(fa.ctypes.data_as(C.c_void_p), fb.ctypes.data_as(C.c_void_p), C.c_size_t(n))
            assert got == int(want), (n, kind, hex(got), hex(int(want)))
            cases += 1
    assert cases == 42


def test_gaudi3_wide_operand_restatement_matches_reference(hc, ref):
    """fp32 (one sliced MAC per tree) and tf32 (two sliced MACs per tree) against fma_vec of the compiled reference."""
    rng = np.random.default_rng(43)
    hc.hc_g3_dot_fp32.restype = C.c_uint32
    hc.hc_g3_dot_tf32.restype = C.c_uint32
    special = np.array([0, 0x80000000, 1, 0x80000001, 0x007FFFFF, 0x00800000, 0x7F7FFFFF, 0x7F800000, 0xFF800000, 0x7FC00000, 0x7F800001,
                        0x7F80FF00, 0x3F800000, 0xBF800000, 0x00000100, 0x00010000], np.uint32)
    for n in (1, 2, 3, 8, 65, 400):
        for kind in range(4):
            a = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32)
            b = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32)
            if kind >= 1:   # moderate exponents so that sums stay finite and cancel
                a = (a & 0x807FFFFF) | (rng.integers(100, 150, n).astype(np.uint32) << 23)
                b = (b & 0x807FFFFF) | (rng.integers(100, 150, n).astype(np.uint32) << 23)
            if kind == 2:   # denormals and zeros mixed in
                a[::3] &= 0x807FFFFF
                b[1::4] &= 0x80000000
            if kind == 3:   # every special pattern
                a[: min(n, special.size)] = special[: min(n, special.size)]
                b[: min(n, special.size)] = special[::-1][: min(n, special.size)]
            want = np.float32(ref.fma_vec(abi.FP32, abi.FP32, a, b)).view(np.uint32)
            got = hc.hc_g3_dot_fp32(a.ctypes.data_as(C.c_void_p), b.ctypes.data_as(C.c_void_p), C.c_size_t(n))
            assert got == int(want), ("fp32", n, kind, hex(got), hex(int(want)))
            for at, bt in ((a & 0xFFFFE000, b & 0xFFFFE000), (a, b)):   # tf32 values, and fp32 values the chip rounds to tf32 first
                want = np.float32(ref.fma_vec(abi.TF32, abi.TF32, at, bt)).view(np.uint32)
                got = hc.hc_g3_dot_tf32(at.ctypes.data_as(C.c_void_p), bt.ctypes.data_as(C.c_void_p), C.c_size_t(n))
                assert got == int(want), ("tf32", n, kind, hex(got), hex(int(want)))
