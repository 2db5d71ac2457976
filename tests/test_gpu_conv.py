"""GPU parity of convolution forward / dedx / dedw through the C ABI against the CPU oracle: the
general lowering (any geometry) and the implicit-GEMM path (im2col-mode TMA) on the same inputs."""
import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util
from golden.make_golden import CONV_CASES, conv_shapes

pytestmark = pytest.mark.gpu
OPS = ((abi.OP_FWD, "fwd"), (abi.OP_DEDX, "dedx"), (abi.OP_DEDW, "dedw"))


def make_inputs(rng, c, dtype=abi.BF16, port=None):
    xs, ws, ys = conv_shapes(c)
    if dtype == abi.BF16:
        xb = util.gen_bf16(rng, int(np.prod(xs)), "normal")
        wb = util.gen_bf16(rng, int(np.prod(ws)), "normal", 0.05)
        yb = util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.01)
        kw = {}
    else:
        xb, wb, yb = (util.gen_fp8(rng, int(np.prod(s)), port) for s in (xs, ws, ys))
        kw = dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL)
    return (xs, ws, ys), (T(xb, dtype, xs, **kw), T(wb, dtype, ws, **kw), T(yb, dtype, ys, **kw)), (xb, wb, yb)


def check_all_ops(calc, oracle, c, dim=2, dtype=abi.BF16, port=None, seed=0):
    """Every output of fwd / dedx / dedw against the oracle, per element: |gpu - ref| <= 1e-5 * sum|a_k b_k|, the sum
    taken from the same convolution on the operands' absolute values."""
    rng = np.random.default_rng(seed)
    shapes, (x, w, y), bits = make_inputs(rng, c, dtype, port)
    xs, ws, ys = shapes
    kw = {} if dtype == abi.BF16 else dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL)
    cp = abi.make_conv_params(dim, c[8], c[7], c[9])
    for op, nm in OPS:
        shp = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[op]
        o1, o2 = np.full(int(np.prod(shp)), 3.0, np.float32), np.full(int(np.prod(shp)), 3.0, np.float32)
        calc.do_convolution(T(o1, abi.FP32, shp), x, w, y, cp, op)
        assert oracle.conv(T(o2, abi.FP32, shp), x, w, y, cp, op) == 0
        util.assert_acc(o1, o2, util.conv_sum_abs(oracle, shapes, bits, dtype, cp, op, **kw), "%s %s" % (nm, c))


@pytest.mark.parametrize("c", CONV_CASES + [
    (16, 24, 12, 10, 3, 3, 3, (2, 2), (1, 1), (1, 1)),
    (3, 8, 15, 11, 2, 5, 3, (1, 1), (2, 1), (1, 1)),
    (24, 16, 8, 8, 2, 1, 1, (1, 1), (0, 0), (1, 1)),
])
def test_general_lowering(calc, best_oracle, c):
    check_all_ops(calc, best_oracle, c)


@pytest.mark.parametrize("c", [
    (64, 64, 32, 32, 2, 3, 3, (1, 1), (1, 1), (1, 1)),
    (128, 64, 30, 34, 2, 3, 3, (1, 1), (1, 1), (1, 1)),
    (64, 128, 33, 31, 2, 3, 2, (2, 2), (1, 1), (1, 1)),
    (64, 64, 40, 36, 1, 3, 3, (1, 1), (2, 2), (2, 2)),
    (192, 80, 20, 24, 3, 1, 1, (1, 1), (0, 0), (1, 1)),
    (64, 72, 37, 29, 2, 5, 5, (1, 1), (2, 2), (1, 1)),
])
def test_implicit_gemm_path(calc, best_oracle, c):
    """Geometries the im2col-mode TMA path takes (2-D, C a multiple of 64, activations over 128 KiB)."""
    check_all_ops(calc, best_oracle, c, seed=1)


@pytest.mark.parametrize("c", [
    (64, 128, 33, 31, 2, 3, 2, (2, 2), (1, 1), (1, 1)),      # 2 x 2 parity classes with 2/1 x 1/1 taps
    (64, 64, 40, 36, 2, 3, 3, (2, 2), (1, 1), (1, 1)),       # the ResNet down-sampling geometry
    (128, 64, 41, 37, 2, 5, 5, (3, 2), (2, 2), (2, 1)),      # stride 3 x 2 with dilation 2 x 1: some classes see no tap in one dim
    (64, 256, 48, 44, 2, 1, 1, (2, 2), (0, 0), (1, 1)),      # 1 x 1 filter: three of the four classes stay zero
    (64, 64, 39, 35, 3, 4, 3, (2, 3), (0, 1), (1, 2)),       # odd extents: the last dX rows lie beyond the last tap
])
def test_strided_dedx_runs_as_implicit_gemm_per_parity_class(calc, best_oracle, c):
    """dedx of a strided convolution on the implicit-GEMM path (one launch per parity class of dX positions, no column
    matrix): every output against the oracle, positions no tap reaches included (they must be zero)."""
    rng = np.random.default_rng(11)
    shapes, (x, w, y), bits = make_inputs(rng, c)
    xs, ws, ys = shapes
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    o1, o2 = np.full(int(np.prod(xs)), 3.0, np.float32), np.full(int(np.prod(xs)), 3.0, np.float32)
    before = calc.launch_count()
    calc.do_convolution(T(o1, abi.FP32, xs), x, w, y, cp, abi.OP_DEDX)
    launches = calc.launch_count() - before
    assert launches <= c[7][0] * c[7][1], launches      # at most one GEMM per class: no im2col / col2im kernels ran
    assert best_oracle.conv(T(o2, abi.FP32, xs), x, w, y, cp, abi.OP_DEDX) == 0
    util.assert_acc(o1, o2, util.conv_sum_abs(best_oracle, shapes, bits, abi.BF16, cp, abi.OP_DEDX), "strided dedx %s" % (c,))
    assert ((o2 == 0) <= (o1 == 0)).all()                # where the reference left its zero fill, so did we
    # the fused bf16 cast writes the same sub-grids
    o16 = np.full(int(np.prod(xs)), 0x1234, np.uint16)
    calc.do_convolution(T(o16, abi.BF16, xs), x, w, y, cp, abi.OP_DEDX, abi.RM_NE, abi.make_cast_params(abi.RM_NE))
    assert (o16 == util.f32_to_bf16_rne(o1)).all()


@pytest.mark.parametrize("pair", [1, 0])
def test_implicit_gemm_wide_channels_on_both_kernels(calc, best_oracle, pair):
    """256 channels in and out: all three operations qualify for the CTA-pair kernel (pair = 1); pair = 0 forces
    the single-CTA kernel on the same problem."""
    calc.set_option("pair", pair)
    try:
        check_all_ops(calc, best_oracle, (256, 256, 20, 18, 2, 3, 3, (1, 1), (1, 1), (1, 1)), seed=3)
        check_all_ops(calc, best_oracle, (256, 320, 17, 19, 1, 3, 3, (1, 1), (1, 1), (2, 2)), seed=4)
    finally:
        calc.set_option("pair", -1)


def test_implicit_gemm_fp8(calc, best_oracle, port):
    check_all_ops(calc, best_oracle, (128, 128, 32, 32, 2, 3, 3, (1, 1), (1, 1), (1, 1)), dtype=abi.FP8_143, port=port, seed=2)


def test_3d_convolution(calc, best_oracle):
    rng = np.random.default_rng(6)
    cp = abi.make_conv_params(3, (1, 1, 1), (1, 1, 1), (1, 1, 1))
    xs, ws, ys = [4, 5, 5, 4, 2], [3, 4, 2, 2, 2], [3, 6, 6, 5, 2]
    xb, wb, yb = util.gen_bf16(rng, int(np.prod(xs)), "normal"), util.gen_bf16(rng, int(np.prod(ws)), "normal", 0.1), util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.01)
    x, w, y = T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), T(yb, abi.BF16, ys)
    for op, shp in ((abi.OP_FWD, ys), (abi.OP_DEDX, xs), (abi.OP_DEDW, ws)):
        o1, o2 = np.zeros(int(np.prod(shp)), np.float32), np.zeros(int(np.prod(shp)), np.float32)
        calc.do_convolution(T(o1, abi.FP32, shp), x, w, y, cp, op)
        assert best_oracle.conv(T(o2, abi.FP32, shp), x, w, y, cp, op) == 0
        util.assert_acc(o1, o2, util.conv_sum_abs(best_oracle, (xs, ws, ys), (xb, wb, yb), abi.BF16, cp, op), "3-D conv op %d" % op)


def test_golden_convolutions(calc, golden, port):
    for i, c in enumerate(CONV_CASES):
        shapes = conv_shapes(c)
        xs, ws, ys = shapes
        cp = abi.make_conv_params(2, c[8], c[7], c[9])
        bits = (golden["conv%d_x" % i], golden["conv%d_w" % i], golden["conv%d_y" % i])
        x, w, y = T(bits[0], abi.BF16, xs), T(bits[1], abi.BF16, ws), T(bits[2], abi.BF16, ys)
        for op, nm in OPS:
            shp = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[op]
            o = np.full(int(np.prod(shp)), 3.0, np.float32)
            calc.do_convolution(T(o, abi.FP32, shp), x, w, y, cp, op)
            util.assert_acc(o, golden["conv%d_%s" % (i, nm)], util.conv_sum_abs(port, shapes, bits, abi.BF16, cp, op), "golden conv %d %s" % (i, nm))


def test_dedx_strided_leaves_untouched_positions_zero(calc, best_oracle):
    # stride 2 with a 1x1 filter: three of four dx positions receive nothing (im2col.cpp:106 zero-fills)
    c = (8, 8, 8, 8, 1, 1, 1, (2, 2), (0, 0), (1, 1))
    rng = np.random.default_rng(3)
    (xs, ws, ys), (x, w, y), _ = make_inputs(rng, c)
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    o = np.full(int(np.prod(xs)), 9.0, np.float32)
    calc.do_convolution(T(o, abi.FP32, xs), x, w, y, cp, abi.OP_DEDX)
    img = o.reshape(8, 8, 8)  # (H, W, C)
    assert (img[1::2] == 0).all() and (img[:, 1::2] == 0).all() and (img[::2, ::2] != 0).any()


def test_dedx_rounding_mode_reaches_the_tap_adds(calc, best_oracle):
    c = (8, 6, 7, 6, 2, 3, 3, (1, 1), (1, 1), (1, 1))
    rng = np.random.default_rng(4)
    shapes, (x, w, y), bits = make_inputs(rng, c)
    xs, ws, ys = shapes
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    sabs = util.conv_sum_abs(best_oracle, shapes, bits, abi.BF16, cp, abi.OP_DEDX)
    for rm in (abi.RM_Z, abi.RM_UP, abi.RM_DOWN):
        o1, o2 = np.zeros(int(np.prod(xs)), np.float32), np.zeros(int(np.prod(xs)), np.float32)
        calc.do_convolution(T(o1, abi.FP32, xs), x, w, y, cp, abi.OP_DEDX, rm)
        assert best_oracle.conv(T(o2, abi.FP32, xs), x, w, y, cp, abi.OP_DEDX, rm) == 0
        util.assert_acc(o1, o2, sabs, "dedx rm %d" % rm)


def test_fused_bf16_output(calc, best_oracle, port):
    """conv fwd with a fused RNE bf16 cast (the ResNet-shaped forward convolution's output type): <= 1 ulp, or within the
    accumulator tolerance for near-cancellation outputs."""
    c = (64, 64, 32, 32, 2, 3, 3, (1, 1), (1, 1), (1, 1))
    rng = np.random.default_rng(5)
    (xs, ws, ys), (x, w, y), (xb, wb, yb) = make_inputs(rng, c)
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    n = int(np.prod(ys))
    out = np.zeros(n, np.uint16)
    calc.do_convolution(T(out, abi.BF16, ys), x, w, y, cp, abi.OP_FWD, abi.RM_NE, abi.make_cast_params(abi.RM_NE))
    acc = np.zeros(n, np.float32)
    assert best_oracle.conv(T(acc, abi.FP32, ys), x, w, y, cp, abi.OP_FWD) == 0
    ref = port.fp32_to_bf16(acc)
    # sum|ab| per output via the same convolution on absolute values (exact enough in fp32 on the GPU)
    ax, aw = T(xb & 0x7FFF, abi.BF16, xs), T(wb & 0x7FFF, abi.BF16, ws)
    sabs = np.zeros(n, np.float32)
    calc.do_convolution(T(sabs, abi.FP32, ys), ax, aw, y, cp, abi.OP_FWD)
    inexact, far = util.check_rounded(out, ref, 16, util.bf16_to_f32(out), util.bf16_to_f32(ref), sabs.astype(np.float64), "conv fwd bf16")
    assert inexact < 0.02 * n


def test_transposed_dedx(calc, golden, port):
    """transposed_dedx == dedx on weights with their two fastest dims swapped and S mirrored; checked
    against the reference's own output (golden) and against dedx on host-flipped weights (bit-identical)."""
    c = CONV_CASES[0]
    xs, ws, ys = conv_shapes(c)
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    wt_shape = [ws[1], ws[0], ws[2], ws[3]]
    wt = golden["tdedx_w"]
    x, y = T(golden["conv0_x"], abi.BF16, xs), T(golden["conv0_y"], abi.BF16, ys)
    o = np.zeros(int(np.prod(xs)), np.float32)
    calc.do_convolution(T(o, abi.FP32, xs), x, T(wt, abi.BF16, wt_shape), y, cp, abi.OP_TRANSPOSED_DEDX)
    # sum|ab| of dedx: the same operation on the absolute values of dY and of the weights in dedx layout
    w4 = wt.reshape(wt_shape[3], wt_shape[2], wt_shape[1], wt_shape[0])          # (R, S, i1, i0)
    flipped = np.ascontiguousarray(w4[:, ::-1].transpose(0, 1, 3, 2))               # (R, S', i0, i1) -> [K, C, S, R] memory
    sabs = util.conv_sum_abs(port, (xs, ws, ys), (golden["conv0_x"], flipped.reshape(-1), golden["conv0_y"]), abi.BF16, cp, abi.OP_DEDX)
    util.assert_acc(o, golden["tdedx_out"], sabs, "transposed dedx")
    o2 = np.zeros(int(np.prod(xs)), np.float32)
    calc.do_convolution(T(o2, abi.FP32, xs), x, T(flipped, abi.BF16, ws), y, cp, abi.OP_DEDX)
    assert (o.view(np.uint32) == o2.view(np.uint32)).all()


def test_errors(calc):
    a = np.zeros(4096, np.uint16)
    cp = abi.make_conv_params(2)
    with pytest.raises(pkg.MmeError):  # output shape is not y's shape
        calc.do_convolution(T(np.zeros(10, np.float32), abi.FP32, [2, 5, 1, 1]), T(a, abi.BF16, [4, 4, 4, 1]), T(a, abi.BF16, [2, 4, 1, 1]),
                            T(a, abi.BF16, [2, 4, 4, 1]), cp, abi.OP_FWD)
    with pytest.raises(pkg.MmeError) as ei:   # integer activations: outside this backend, never a CPU result
        calc.do_convolution(T(np.zeros(32, np.float32), abi.FP32, [2, 4, 4, 1]), T(a, 2, [4, 4, 4, 1]), T(a, 2, [2, 4, 1, 1]),
                            T(a, 2, [2, 4, 4, 1]), cp, abi.OP_FWD)
    assert ei.value.status == abi.ERR_UNSUPPORTED
