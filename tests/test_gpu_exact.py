"""The bit-exact accumulation mode (mmeb200_set_accumulation(MMEB200_ACC_CHIP_EXACT)): accumulators, and everything
downstream of them, must equal the reference's Gaudi3 model bit for bit -- GEMM in every orientation, fp8 with every
bias / Inf-NaN convention (random codes, so Inf and NaN occur), the rounded cast including the LFSR stochastic stream,
and the three convolutions."""
import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util
from golden.make_golden import CONV_CASES, GEMM_CASES, conv_shapes

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def exact():
    c = pkg.Calculator(device=0)
    c.set_accumulation(abi.ACC_CHIP_EXACT)
    yield c
    c.close()


def bits(a):
    return a.view(np.uint32)


@pytest.mark.parametrize("op", [abi.OP_AB, abi.OP_ABT, abi.OP_ATB, abi.OP_ATBT])
def test_bf16_gemm_bit_exact(exact, best_oracle, op):
    rng = np.random.default_rng(op)
    for (M, N, K, batch, xb_dims, wb_dims) in ((70, 129, 203, (), None, None), (64, 64, 8, (3, 2), (3, 1), (1, 2)), (5, 3, 1, (), None, None),
                                               (200, 96, 1000, (2,), None, None)):
        tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
        xbd = list(batch if xb_dims is None else xb_dims)
        wbd = list(batch if wb_dims is None else wb_dims)
        xs = ([M, K] if tA else [K, M]) + xbd
        ws = ([K, N] if tB else [N, K]) + wbd
        os_ = [N, M] + list(batch)
        # wide exponent spread: alignment and truncation matter
        xb = util.gen_bf16(rng, int(np.prod(xs)), "normal") ^ (rng.integers(0, 2, int(np.prod(xs))).astype(np.uint16) << 9)
        wb = util.gen_bf16(rng, int(np.prod(ws)), "normal", 50.0)
        o1, o2 = np.full(int(np.prod(os_)), 7.0, np.float32), np.full(int(np.prod(os_)), 7.0, np.float32)
        exact.do_batch_gemm(T(o1, abi.FP32, os_), T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), op)
        assert best_oracle.bgemm(T(o2, abi.FP32, os_), T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), op) == 0
        assert (bits(o1) == bits(o2)).all(), (op, M, N, K, int((bits(o1) != bits(o2)).sum()))


@pytest.mark.parametrize("tx,tw,bx,bw,mx,mw", [(9, 9, 7, 7, 2, 2), (9, 9, 3, 15, 2, 0), (10, 9, 15, 11, 0, 2), (10, 10, 20, 1, 1, 0), (9, 10, 15, 30, 1, 2)])
def test_fp8_gemm_bit_exact_on_random_codes(exact, best_oracle, tx, tw, bx, bw, mx, mw):
    rng = np.random.default_rng(tx * 31 + bw)
    M, N, K = 96, 80, 333
    xb, wb = rng.integers(0, 256, M * K).astype(np.uint8), rng.integers(0, 256, K * N).astype(np.uint8)
    x, w = T(xb, tx, [K, M], fp_bias=bx, inf_nan_mode=mx), T(wb, tw, [N, K], fp_bias=bw, inf_nan_mode=mw)
    o1, o2 = np.zeros(M * N, np.float32), np.zeros(M * N, np.float32)
    exact.do_batch_gemm(T(o1, abi.FP32, [N, M]), x, w, abi.OP_AB)
    assert best_oracle.bgemm(T(o2, abi.FP32, [N, M]), x, w, abi.OP_AB) == 0
    assert (bits(o1) == bits(o2)).all(), int((bits(o1) != bits(o2)).sum())
    if mx == 2 and mw == 2:
        assert np.isnan(o2).any()        # the NaN codes took the general routine
    # finite codes only: the fast routine alone
    xb2, wb2 = xb & 0x77, wb & 0x77
    x2, w2 = T(xb2, tx, [K, M], fp_bias=bx, inf_nan_mode=mx), T(wb2, tw, [N, K], fp_bias=bw, inf_nan_mode=mw)
    exact.do_batch_gemm(T(o1, abi.FP32, [N, M]), x2, w2, abi.OP_AB)
    assert best_oracle.bgemm(T(o2, abi.FP32, [N, M]), x2, w2, abi.OP_AB) == 0
    assert np.isfinite(o2).all() and (bits(o1) == bits(o2)).all()


@pytest.mark.parametrize("dtype", [abi.FP32, abi.TF32])
def test_fp32_and_tf32_gemm_bit_exact(exact, ref, dtype):
    """fp32 / tf32 operands go through the chip's sliced multiplier (one or two MACs per tree); only the compiled reference
    models them, so this needs it."""
    rng = np.random.default_rng(dtype)
    for op, (M, N, K) in ((abi.OP_AB, (40, 33, 77)), (abi.OP_ABT, (17, 20, 64)), (abi.OP_ATB, (9, 50, 131)), (abi.OP_ATBT, (32, 16, 5))):
        tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
        xs, ws = ([M, K] if tA else [K, M]), ([K, N] if tB else [N, K])
        a = (rng.normal(0, 1, M * K) * 10.0 ** rng.integers(-3, 4, M * K)).astype(np.float32)
        b = (rng.normal(0, 1, K * N) * 10.0 ** rng.integers(-3, 4, K * N)).astype(np.float32)
        a[:4] = [0.0, -0.0, 1e-40, np.inf]
        if dtype == abi.TF32:
            a, b = (a.view(np.uint32) & 0xFFFFE000).view(np.float32), (b.view(np.uint32) & 0xFFFFE000).view(np.float32)
        o1, o2 = np.zeros(M * N, np.float32), np.zeros(M * N, np.float32)
        exact.do_batch_gemm(T(o1, abi.FP32, [N, M]), T(a, dtype, xs), T(b, dtype, ws), op)
        assert ref.bgemm(T(o2, abi.FP32, [N, M]), T(a, dtype, xs), T(b, dtype, ws), op) == 0
        assert (bits(o1) == bits(o2)).all(), (dtype, op, int((bits(o1) != bits(o2)).sum()))


def test_cast_after_exact_accumulation_is_bit_exact_including_stochastic_rounding(exact, port, best_oracle):
    rng = np.random.default_rng(8)
    M, N, K = 130, 70, 96
    xb, wb = util.gen_bf16(rng, M * K, "normal"), util.gen_bf16(rng, K * N, "normal")
    x, w = T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, [N, K])
    acc = np.zeros(M * N, np.float32)
    assert best_oracle.bgemm(T(acc, abi.FP32, [N, M]), x, w, abi.OP_AB) == 0
    regs = np.arange(5, 261, dtype=np.uint32)
    for od, bias, mode, rm in ((abi.BF16, 0, 0, abi.RM_NE), (abi.BF16, 0, 0, abi.RM_SR), (abi.FP8_143, 7, 2, abi.RM_SR), (abi.FP8_152, 15, 0, abi.RM_NE)):
        cp = abi.make_cast_params(rm, clip_fp=True)
        want = np.zeros(M * N, abi.NP_DTYPE[od])
        rc, _ = port.activation(T(want, od, [N, M], fp_bias=bias, inf_nan_mode=mode), T(acc.copy(), abi.FP32, [N, M]), cp, regs.copy(), 41)
        assert rc == 0
        got = np.zeros(M * N, abi.NP_DTYPE[od])
        exact.set_lfsr(regs, 41)
        exact.do_batch_gemm(T(got, od, [N, M], fp_bias=bias, inf_nan_mode=mode), x, w, abi.OP_AB, cp)
        assert (got == want).all(), (od, rm, int((got != want).sum()))


@pytest.mark.parametrize("c", [
    (16, 24, 12, 10, 2, 3, 3, (1, 1), (1, 1), (1, 1)),
    (64, 64, 20, 18, 2, 3, 3, (1, 1), (1, 1), (1, 1)),      # a geometry the tensor-core mode would run through im2col-mode TMA
    (24, 16, 15, 11, 2, 5, 3, (2, 1), (2, 1), (1, 2)),
    (8, 8, 8, 8, 1, 1, 1, (2, 2), (0, 0), (1, 1)),
])
def test_convolutions_bit_exact(exact, best_oracle, c):
    rng = np.random.default_rng(c[0] + c[5])
    xs, ws, ys = conv_shapes(c)
    xb = util.gen_bf16(rng, int(np.prod(xs)), "normal")
    wb = util.gen_bf16(rng, int(np.prod(ws)), "normal", 0.05)
    yb = util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.01)
    x, w, y = T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), T(yb, abi.BF16, ys)
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    for op, shp in ((abi.OP_FWD, ys), (abi.OP_DEDX, xs), (abi.OP_DEDW, ws)):
        o1, o2 = np.full(int(np.prod(shp)), 3.0, np.float32), np.full(int(np.prod(shp)), 3.0, np.float32)
        exact.do_convolution(T(o1, abi.FP32, shp), x, w, y, cp, op)
        assert best_oracle.conv(T(o2, abi.FP32, shp), x, w, y, cp, op) == 0
        assert (bits(o1) == bits(o2)).all(), (op, c, int((bits(o1) != bits(o2)).sum()))


def test_committed_golden_outputs_are_reproduced_bit_for_bit(exact, golden):
    """tests/golden/golden_small.npz holds outputs of the compiled reference (Gaudi3 model: chip 2); no oracle is needed here."""
    for i, (M, N, K, op, batch) in enumerate(GEMM_CASES):
        tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
        xs = ([M, K] if tA else [K, M]) + list(batch)
        ws = ([K, N] if tB else [N, K]) + list(batch)
        want = golden["gemm%d_chip2" % i]
        o = np.zeros(want.size, np.float32)
        exact.do_batch_gemm(T(o, abi.FP32, [N, M] + list(batch)), T(golden["gemm%d_x" % i], abi.BF16, xs), T(golden["gemm%d_w" % i], abi.BF16, ws), op)
        assert (bits(o) == bits(np.ascontiguousarray(want, np.float32))).all(), ("gemm", i)
    M, N, K = 16, 24, 40
    for j, (tx, tw, bx, bw, mx, mw) in enumerate(((9, 9, 7, 11, 2, 2), (10, 9, 15, 7, 0, 2), (9, 10, 3, 20, 1, 1), (9, 9, 15, 15, 0, 0))):
        o = np.zeros(M * N, np.float32)
        exact.do_batch_gemm(T(o, abi.FP32, [N, M]), T(golden["fp8gemm_x"], tx, [K, M], fp_bias=bx, inf_nan_mode=mx),
                            T(golden["fp8gemm_w"], tw, [N, K], fp_bias=bw, inf_nan_mode=mw), abi.OP_AB)
        assert (bits(o) == golden["fp8gemm_%d" % j]).all(), ("fp8", j)
    for dt, nm in ((abi.FP32, "fp32"), (abi.TF32, "tf32")):
        o = np.zeros(M * N, np.float32)
        exact.do_batch_gemm(T(o, abi.FP32, [N, M]), T(golden["f32gemm_x"], dt, [K, M]), T(golden["f32gemm_w"], dt, [N, K]), abi.OP_AB)
        assert (bits(o) == bits(np.ascontiguousarray(golden["f32gemm_" + nm], np.float32))).all(), nm
    for i, c in enumerate(CONV_CASES):
        xs, ws, ys = conv_shapes(c)
        cp = abi.make_conv_params(2, c[8], c[7], c[9])
        if i == 0:
            o = np.zeros(int(np.prod(xs)), np.float32)
            exact.do_convolution(T(o, abi.FP32, xs), T(golden["conv0_x"], abi.BF16, xs), T(golden["tdedx_w"], abi.BF16, [ws[1], ws[0], ws[2], ws[3]]),
                                 T(golden["conv0_y"], abi.BF16, ys), cp, abi.OP_TRANSPOSED_DEDX)
            assert (bits(o) == bits(np.ascontiguousarray(golden["tdedx_out"], np.float32))).all(), "transposed_dedx"
        x, w, y = T(golden["conv%d_x" % i], abi.BF16, xs), T(golden["conv%d_w" % i], abi.BF16, ws), T(golden["conv%d_y" % i], abi.BF16, ys)
        for op, nm, shp in ((abi.OP_FWD, "fwd", ys), (abi.OP_DEDX, "dedx", xs), (abi.OP_DEDW, "dedw", ws)):
            want = np.ascontiguousarray(golden["conv%d_%s" % (i, nm)], np.float32)
            o = np.full(want.size, 3.0, np.float32)
            exact.do_convolution(T(o, abi.FP32, shp), x, w, y, cp, op)
            assert (bits(o) == bits(want)).all(), ("conv", i, nm)


def test_mode_rules(calc):
    c2 = pkg.Calculator(chip=abi.CHIP_GAUDI2)
    with pytest.raises(Exception, match="Gaudi3"):
        c2.set_accumulation(abi.ACC_CHIP_EXACT)
    c2.close()
    c3 = pkg.Calculator()
    c3.set_accumulation(abi.ACC_CHIP_EXACT)
    a = np.ones(64, np.float32)
    h = np.full(64, 0x3F80, np.uint16)
    o = np.zeros(64, np.float32)
    with pytest.raises(Exception, match="bit-exact accumulation takes"):
        c3.do_batch_gemm(T(o, abi.FP32, [8, 8]), T(h, abi.BF16, [8, 8]), T(a, abi.FP32, [8, 8]), abi.OP_AB)
    c3.do_batch_gemm(T(o, abi.FP32, [8, 8]), T(a, abi.FP32, [8, 8]), T(a, abi.FP32, [8, 8]), abi.OP_AB)
    assert (o == 8.0).all()
    c3.set_accumulation(abi.ACC_TENSOR_CORE)
    o[:] = 0
    c3.do_batch_gemm(T(o, abi.FP32, [8, 8]), T(a, abi.FP32, [8, 8]), T(a, abi.FP32, [8, 8]), abi.OP_AB)
    assert (o == 8.0).all()
    c3.close()
