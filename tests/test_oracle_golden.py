"""Pins the CPU restatement (oracle/mme_oracle.c) against the reference's own known-answer unit
tests (mme/tests/unit_tests/mme_unit_test.cpp) and against golden vectors produced by running the
unmodified reference (tests/golden/make_golden.py). Runs without a GPU and without the reference."""
import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util
from golden.make_golden import CONV_CASES, GEMM_CASES, conv_shapes


def f32(x):
    return np.array([x], dtype=np.float32)


# ---- known answers of mme_unit_test.cpp ---------------------------------------------------------
def test_fp8_143_convert_known_answer(port):
    # mme_unit_test.cpp:394-408: -0.25 -> 0x88 at bias 3, and back
    code = port.fp32_to_fp8(f32(-0.25), 4, 3, abi.RM_NE)
    assert code[0] == 0x88
    assert port.fp8_to_fp32(code, 4, 3, 0)[0] == np.float32(-0.25)


def test_fp8_152_convert_known_answer(port):
    # mme_unit_test.cpp:467-481: -0.5 -> 0xB8 at bias 15, and back
    code = port.fp32_to_fp8(f32(-0.5), 5, 15, abi.RM_NE)
    assert code[0] == 0xB8
    assert port.fp8_to_fp32(code, 5, 15, 0)[0] == np.float32(-0.5)


def test_fp8_products_known_answer(port):
    # mme_unit_test.cpp:410-423,483-496
    a = port.fp8_to_fp32(port.fp32_to_fp8(f32(0.25), 4, 15), 4, 15, 0)[0]
    b = port.fp8_to_fp32(port.fp32_to_fp8(f32(-0.5), 4, 15), 4, 15, 0)[0]
    assert a * b == np.float32(0.25 * -0.5)
    a = port.fp8_to_fp32(port.fp32_to_fp8(f32(0.5), 5, 15), 5, 15, 0)[0]
    b = port.fp8_to_fp32(port.fp32_to_fp8(f32(-0.5), 5, 15), 5, 15, 0)[0]
    assert a * b == np.float32(-0.25)


def test_bf16_conversions_known_answer(port):
    # mme_unit_test.cpp:13-29: max bf16 0x7f7f is finite, 0x7f80 is +Inf, 0 is zero
    assert util.bf16_to_f32(np.array([0x7F7F], np.uint16))[0] == np.array([0x7F7F0000], np.uint32).view(np.float32)[0]
    assert np.isinf(util.bf16_to_f32(np.array([0x7F80], np.uint16))[0])
    assert port.fp32_to_bf16(f32(10.0))[0] == 0x4120


def test_gemm_1x5_bf16_known_answer(port):
    # mme_unit_test.cpp:108-125: [1x5] of 10 times [5x1] of 10 = 500
    ten = port.fp32_to_bf16(np.full(5, 10.0, np.float32))
    y = np.zeros(1, np.float32)
    assert port.bgemm(T(y, abi.FP32, [1, 1]), T(ten, abi.BF16, [5, 1]), T(ten, abi.BF16, [1, 5]), abi.OP_AB) == 0
    assert y[0] == 500.0


def test_gemm_5x5_bf16_with_activation_known_answer(port):
    # mme_unit_test.cpp:147-172: 5x5 of 10 times 5x5 of 5 = 250 everywhere, also after the bf16 cast
    a = port.fp32_to_bf16(np.full(25, 10.0, np.float32))
    b = port.fp32_to_bf16(np.full(25, 5.0, np.float32))
    acc = np.zeros(25, np.float32)
    assert port.bgemm(T(acc, abi.FP32, [5, 5]), T(a, abi.BF16, [5, 5]), T(b, abi.BF16, [5, 5]), abi.OP_AB) == 0
    assert (acc == 250.0).all()
    y = np.zeros(25, np.uint16)
    rc, _ = port.activation(T(y, abi.BF16, [5, 5]), T(acc, abi.FP32, [5, 5]), abi.make_cast_params(), np.arange(2, 258), 37)
    assert rc == 0 and (util.bf16_to_f32(y) == 250.0).all()


@pytest.mark.parametrize("dtype,ew,bias,va,vb", [(abi.FP8_143, 4, 7, 0.25, -0.5), (abi.FP8_152, 5, 15, 0.5, -0.5)])
def test_gemm_2_element_fp8_known_answer(port, dtype, ew, bias, va, vb):
    # mme_unit_test.cpp:425-447,498-519: two-element dot product = 2 * a * b
    a = np.repeat(port.fp32_to_fp8(f32(va), ew, bias), 2)
    b = np.repeat(port.fp32_to_fp8(f32(vb), ew, bias), 2)
    y = np.zeros(1, np.float32)
    assert port.bgemm(T(y, abi.FP32, [1, 1]), T(a, dtype, [2, 1], fp_bias=bias), T(b, dtype, [1, 2], fp_bias=bias), abi.OP_AB) == 0
    assert y[0] == np.float32(va * vb * 2)


# ---- golden vectors from the compiled reference --------------------------------------------------
def test_decode_matches_golden(port, golden):
    codes = np.arange(256, dtype=np.uint8)
    for ew, biases in ((4, (3, 7, 11, 15)), (5, (1, 15, 30))):
        for b in biases:
            for mode in (0, 1, 2):
                got = port.fp8_to_fp32(codes, ew, b, mode).view(np.uint32)
                assert (got == golden["dec_%d_%d_%d" % (ew, b, mode)]).all(), (ew, b, mode)


def test_casts_match_golden(port, golden):
    bits, lfsr = golden["cast_in"], golden["cast_lfsr"]
    for rm in (0, 1, 2, 3, 4, 6, 7):
        assert (port.fp32_to_bf16(bits, rm, lfsr) == golden["bf16_rm%d" % rm]).all()
        assert (port.fp32_to_bf16(bits, rm, lfsr, True, True, False) == golden["bf16_rm%d_clip_ftz" % rm]).all()
        for ew, b, mode in ((4, 7, 2), (4, 11, 0), (4, 3, 1), (5, 15, 0), (5, 20, 2)):
            assert (port.fp32_to_fp8(bits, ew, b, rm, lfsr, False, False, False, False, mode) ==
                    golden["fp8_%d_%d_%d_rm%d" % (ew, b, mode, rm)]).all(), (ew, b, mode, rm)
            assert (port.fp32_to_fp8(bits, ew, b, rm, lfsr, True, True, False, True, mode) ==
                    golden["fp8_%d_%d_%d_rm%d_flags" % (ew, b, mode, rm)]).all(), (ew, b, mode, rm)


def test_bgemm_matches_golden_bitwise(port, golden):
    for i, (M, N, K, op, batch) in enumerate(GEMM_CASES):
        tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
        xs = ([M, K] if tA else [K, M]) + list(batch)
        ws = ([K, N] if tB else [N, K]) + list(batch)
        o = np.zeros(golden["gemm%d_chip2" % i].size, np.float32)
        assert port.bgemm(T(o, abi.FP32, [N, M] + list(batch)), T(golden["gemm%d_x" % i], abi.BF16, xs),
                          T(golden["gemm%d_w" % i], abi.BF16, ws), op) == 0
        assert (o.view(np.uint32) == golden["gemm%d_chip2" % i].view(np.uint32)).all(), i


def test_fp8_bgemm_matches_golden_bitwise(port, golden):
    M, N, K = 16, 24, 40
    for j, (tx, tw, bx, bw, mx, mw) in enumerate(((9, 9, 7, 11, 2, 2), (10, 9, 15, 7, 0, 2), (9, 10, 3, 20, 1, 1), (9, 9, 15, 15, 0, 0))):
        o = np.zeros(M * N, np.float32)
        assert port.bgemm(T(o, abi.FP32, [N, M]), T(golden["fp8gemm_x"], tx, [K, M], fp_bias=bx, inf_nan_mode=mx),
                          T(golden["fp8gemm_w"], tw, [N, K], fp_bias=bw, inf_nan_mode=mw), abi.OP_AB) == 0
        assert (o.view(np.uint32) == golden["fp8gemm_%d" % j]).all(), j


def test_conv_matches_golden_bitwise(port, golden):
    for i, c in enumerate(CONV_CASES):
        xs, ws, ys = conv_shapes(c)
        cp = abi.make_conv_params(2, c[8], c[7], c[9])
        x, w, y = T(golden["conv%d_x" % i], abi.BF16, xs), T(golden["conv%d_w" % i], abi.BF16, ws), T(golden["conv%d_y" % i], abi.BF16, ys)
        for op, shp, nm in ((abi.OP_FWD, ys, "fwd"), (abi.OP_DEDX, xs, "dedx"), (abi.OP_DEDW, ws, "dedw")):
            o = np.full(int(np.prod(shp)), 3.0, np.float32)
            assert port.conv(T(o, abi.FP32, shp), x, w, y, cp, op) == 0
            assert (o.view(np.uint32) == golden["conv%d_%s" % (i, nm)].view(np.uint32)).all(), (i, nm)


def test_activation_matches_golden(port, golden):
    n = golden["act_acc"].size
    for od, bias, mode, nm in ((abi.BF16, 0, 0, "bf16"), (abi.FP8_143, 7, 2, "f143"), (abi.FP8_152, 15, 0, "f152")):
        for rm in (0, 4, 7):
            for relu in (0, 1):
                o = np.zeros(n, abi.NP_DTYPE[od])
                cp = abi.make_cast_params(rm, relu, clip_fp=(rm == 4))
                rc, _ = port.activation(T(o, od, [n], fp_bias=bias, inf_nan_mode=mode), T(golden["act_acc"].copy(), abi.FP32, [n]),
                                        cp, golden["act_lfsr"].copy(), 37)
                assert rc == 0
                assert (o == golden["act_%s_rm%d_relu%d" % (nm, rm, relu)]).all(), (nm, rm, relu)


def test_zero_common_dim_gives_zeros(port):
    # mme_reference_impl.cpp:204-216
    y = np.full(6, 5.0, np.float32)
    e = np.zeros(1, np.uint16)
    assert port.bgemm(T(y, abi.FP32, [3, 2]), T(e, abi.BF16, [0, 2]), T(e, abi.BF16, [3, 0]), abi.OP_AB) == 0
    assert (y == 0).all()
