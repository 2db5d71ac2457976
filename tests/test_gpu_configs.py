"""The benchmark configurations at their full sizes on the GPU, checked (a) against the CPU oracle on
slices that keep the common dimension whole, so every checked output sees the complete, identically
ordered reduction, and (b) through size-independent properties at full size."""
import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
from intel_gaudi3_software_b200 import workloads as bench
import util

pytestmark = pytest.mark.gpu


def rows_for(oracle, macs_per_row, budget_macs=1.2e9):
    t = max(1, oracle.hardware_threads())
    rows = int(max(8, min(256, budget_macs * min(t, 16) / 8 / macs_per_row)))
    return rows


def test_bf16_gemm_1024_full(calc, best_oracle):
    """The bf16 1024^3 GEMM in full:, uniform[-1,1], fp32 output."""
    rng = np.random.default_rng(1)
    n = 1024
    xb, wb = util.gen_bf16(rng, n * n), util.gen_bf16(rng, n * n)
    x, w = T(xb, abi.BF16, [n, n]), T(wb, abi.BF16, [n, n])
    o = np.zeros(n * n, np.float32)
    calc.do_batch_gemm(T(o, abi.FP32, [n, n]), x, w, abi.OP_AB)
    rows = rows_for(best_oracle, n * n, 4e8)
    r = np.zeros(rows * n, np.float32)
    assert best_oracle.bgemm(T(r, abi.FP32, [n, rows]), T(xb[:rows * n], abi.BF16, [n, rows]), w, abi.OP_AB) == 0
    sabs = util.sum_abs_products(util.bf16_to_f32(xb).reshape(n, n)[:rows], util.bf16_to_f32(wb).reshape(n, n))
    assert util.acc_error(o.reshape(n, n)[:rows], r.reshape(rows, n), sabs) <= util.ACC_TOL
    # full-size property: against float64 on all rows
    ref = util.bf16_to_f32(xb).reshape(n, n).astype(np.float64) @ util.bf16_to_f32(wb).reshape(n, n).astype(np.float64)
    full_sabs = util.sum_abs_products(util.bf16_to_f32(xb).reshape(n, n), util.bf16_to_f32(wb).reshape(n, n))
    assert util.acc_error(o.reshape(n, n), ref, full_sabs) <= util.ACC_TOL


@pytest.mark.parametrize("bias", [7, 11])
def test_fp8_gemm_8192(calc, best_oracle, port, bias):
    """The fp8_143 8192^3 GEMM -> bf16 RNE; bias 11 exercises the exponent-bias fold. Slice = a block
    of A's rows against all of B."""
    wl = dict(bench.WORKLOADS["fp8_gemm_8192"], bias=bias)
    n = 8192
    xb, wb = bench.synth_inputs(wl, seed=2)
    kw = dict(fp_bias=bias, inf_nan_mode=abi.INFNAN_MINIMAL)
    dx, dw, do = calc.to_device(xb), calc.to_device(wb), calc.alloc(n * n * 2)
    calc.do_batch_gemm(T(do.ptr, abi.BF16, [n, n], mem_space=1), T(dx.ptr, abi.FP8_143, [n, n], mem_space=1, **kw),
                       T(dw.ptr, abi.FP8_143, [n, n], mem_space=1, **kw), abi.OP_AB, abi.make_cast_params(abi.RM_NE))
    calc.sync(20_000_000_000)
    out = do.download(np.uint16).reshape(n, n)
    rows = rows_for(best_oracle, n * n)
    pick = np.sort(np.random.default_rng(3).choice(n, rows, replace=False))
    xa = np.ascontiguousarray(xb.reshape(n, n)[pick])
    acc = np.zeros(rows * n, np.float32)
    assert best_oracle.bgemm(T(acc, abi.FP32, [n, rows]), T(xa, abi.FP8_143, [n, rows], **kw), T(wb, abi.FP8_143, [n, n], **kw), abi.OP_AB) == 0
    ref = port.fp32_to_bf16(acc).reshape(rows, n)
    sabs = util.sum_abs_products(util.decode(xa, abi.FP8_143, bias, 2, port).reshape(rows, n), util.decode(wb, abi.FP8_143, bias, 2, port).reshape(n, n))
    inexact, far = util.check_rounded(out[pick], ref, 16, util.bf16_to_f32(out[pick]), util.bf16_to_f32(ref), sabs, "fp8 8192^3")
    assert inexact <= 0.01 * rows * n
    # stochastic rounding (seeded counter-based stream) fused into the epilogue, all 67 M outputs: each is one of the two
    # bf16 neighbours of ITS accumulator (the same launch with an fp32 output gives the accumulators bit for bit: same
    # kernel, same summation order), P(round up) equals the discarded fraction in every fraction bin (5 sigma), and the
    # accumulators themselves are the oracle's within the accumulator tolerance on the sliced rows.
    dacc = calc.alloc(n * n * 4)
    calc.do_batch_gemm(T(dacc.ptr, abi.FP32, [n, n], mem_space=1), T(dx.ptr, abi.FP8_143, [n, n], mem_space=1, **kw),
                       T(dw.ptr, abi.FP8_143, [n, n], mem_space=1, **kw), abi.OP_AB)
    calc.do_batch_gemm(T(do.ptr, abi.BF16, [n, n], mem_space=1), T(dx.ptr, abi.FP8_143, [n, n], mem_space=1, **kw),
                       T(dw.ptr, abi.FP8_143, [n, n], mem_space=1, **kw), abi.OP_AB,
                       abi.make_cast_params(abi.RM_SR, clip_fp=True, rng_kind=abi.RNG_PHILOX, rng_seed=5))
    calc.sync(20_000_000_000)
    gacc = dacc.download(np.float32)
    sr = do.download(np.uint16)
    util.assert_acc(gacc.reshape(n, n)[pick], acc, sabs, "fp8 8192^3 accumulators")
    bits = gacc.view(np.uint32)
    lo = (bits >> 16).astype(np.uint16)
    up = sr != lo
    assert ((sr == lo) | (sr == lo + np.uint16(1))).all()
    frac = (bits & 0xFFFF).astype(np.float64) / 65536.0
    assert not up[frac == 0].any()                      # exactly representable accumulators never move
    for b in range(8):
        sel = (frac >= b / 8) & (frac < (b + 1) / 8)
        p_expect, k = frac[sel].mean(), int(sel.sum())
        assert k > 1_000_000
        assert abs(up[sel].mean() - p_expect) < 5 * np.sqrt(p_expect * (1 - p_expect) / k + 1e-12), (b, up[sel].mean(), p_expect)
    dacc.free()
    for b in (dx, dw, do):
        b.free()


@pytest.mark.parametrize("opname", ["conv_fwd", "conv_dedx", "conv_dedw"])
def test_resnet_conv_full_size(calc, best_oracle, port, opname):
    """The ResNet-shaped convolutions at full size (64 x 56 x 56 x 256, 3x3, 256 -> 256) with the output type the
    configuration names: bf16 round-to-nearest-even for fwd and dedx (cast fused into the epilogue), fp32 for dedw; the fp32
    accumulators of fwd / dedx are checked too. Slices: whole-width strips of the first and the last image for fwd / dedx
    (every checked output sees its complete reduction), channel slices over the full N*H*W reduction for dedw. Rules:
    |acc - ref| <= 1e-5 * sum|a_k b_k| per element, the sum taken from the oracle on the operands' absolute values;
    bf16 outputs <= 1 ulp from the reference's cast of the reference's accumulator, or inside the accumulator rule."""
    wl = bench.WORKLOADS[opname]
    xs, ws, ys = bench.conv_shapes()
    xb, wb, yb = bench.synth_inputs(wl, seed=3)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    op = wl["op"]
    oshape = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[op]
    n_out = int(np.prod(oshape))
    dx, dw, dy = calc.to_device(xb), calc.to_device(wb), calc.to_device(yb)
    do = calc.alloc(n_out * 4)
    tens = (T(dx.ptr, abi.BF16, xs, mem_space=1), T(dw.ptr, abi.BF16, ws, mem_space=1), T(dy.ptr, abi.BF16, ys, mem_space=1))
    calc.do_convolution(T(do.ptr, abi.FP32, oshape, mem_space=1), *tens, cp, op)
    calc.sync(20_000_000_000)
    out = do.download(np.float32)
    img_x, img_y = int(np.prod(xs[:3])), int(np.prod(ys[:3]))
    if op in (abi.OP_FWD, abi.OP_DEDX):
        do16 = calc.alloc(n_out * 2)
        calc.do_convolution(T(do16.ptr, abi.BF16, oshape, mem_space=1), *tens, cp, op, abi.RM_NE, abi.make_cast_params(abi.RM_NE))
        calc.sync(20_000_000_000)
        out16 = do16.download(np.uint16)
        do16.free()
        # crop H to 7 rows at the top border (padding included): rows 0..5 of the crop see the same inputs as in the full image
        Hc = 6
        xs1, ys1 = [xs[0], xs[1], Hc + 1, 1], [ys[0], ys[1], Hc + 1, 1]
        for img in (0, xs[3] - 1):
            xi = xb[img * img_x: img * img_x + int(np.prod(xs1))]
            yi = yb[img * img_y: img * img_y + int(np.prod(ys1))]
            shp = ys1 if op == abi.OP_FWD else xs1
            r = np.zeros(int(np.prod(shp)), np.float32)
            assert best_oracle.conv(T(r, abi.FP32, shp), T(xi, abi.BF16, xs1), T(wb, abi.BF16, ws), T(yi, abi.BF16, ys1), cp, op) == 0
            sabs = util.conv_sum_abs(best_oracle, (xs1, ws, ys1), (xi, wb, yi), abi.BF16, cp, op)
            per_img = img_y if op == abi.OP_FWD else img_x
            cnt = Hc * shp[0] * shp[1]
            got, want, sa = out[img * per_img: img * per_img + cnt], r[:cnt], sabs[:cnt]
            util.assert_acc(got, want, sa, "%s image %d" % (opname, img))
            got16, ref16 = out16[img * per_img: img * per_img + cnt], port.fp32_to_bf16(want)
            inexact, far = util.check_rounded(got16, ref16, 16, util.bf16_to_f32(got16), util.bf16_to_f32(ref16), sa, "%s bf16 image %d" % (opname, img))
            assert inexact <= 0.02 * cnt, (opname, img, inexact, cnt)
    else:
        # dedw: 8 input channels x 8 output channels, all taps, the full 200704-term reduction
        cs, ks = 8, 8
        x4 = xb.reshape(xs[3], xs[2], xs[1], xs[0])[..., :cs].copy()
        y4 = yb.reshape(ys[3], ys[2], ys[1], ys[0])[..., :ks].copy()
        shp = [ks, cs, 3, 3]
        shapes = ([cs, xs[1], xs[2], xs[3]], shp, [ks, ys[1], ys[2], ys[3]])
        r = np.zeros(int(np.prod(shp)), np.float32)
        zw = np.zeros(int(np.prod(shp)), np.uint16)
        assert best_oracle.conv(T(r, abi.FP32, shp), T(x4, abi.BF16, shapes[0]), T(zw, abi.BF16, shp), T(y4, abi.BF16, shapes[2]), cp, op) == 0
        sabs = util.conv_sum_abs(best_oracle, shapes, (x4.reshape(-1), zw, y4.reshape(-1)), abi.BF16, cp, op)
        got = out.reshape(3, 3, ws[1], ws[0])[:, :, :cs, :ks]
        util.assert_acc(got, r.reshape(3, 3, cs, ks), sabs.reshape(3, 3, cs, ks), "conv dedw channel slice")
    for b in (dx, dw, dy, do):
        b.free()


def test_resnet_dedx_stride2_full_size(calc, best_oracle, port):
    """dedx of the 3x3 stride-2 convolution at the ResNet shape (dX 64 x 56 x 56 x 256, dY 64 x 28 x 28 x 256): four implicit
    GEMMs, one per parity class of dX positions, no column matrix (the lowering the reference uses would materialise
    50176 x 2304 fp32 values). Whole first and last image against the oracle, fp32 accumulators and the fused bf16 output."""
    wl = bench.WORKLOADS["conv_dedx_stride2"]
    xs, ws, ys = bench.conv_shapes(wl)
    xb, wb, yb = bench.synth_inputs(wl, seed=4)
    cp = abi.make_conv_params(2, (1, 1), (2, 2), (1, 1))
    n_out = int(np.prod(xs))
    dx, dw, dy = calc.to_device(xb), calc.to_device(wb), calc.to_device(yb)
    do, do16 = calc.alloc(n_out * 4), calc.alloc(n_out * 2)
    tens = (T(dx.ptr, abi.BF16, xs, mem_space=1), T(dw.ptr, abi.BF16, ws, mem_space=1), T(dy.ptr, abi.BF16, ys, mem_space=1))
    before = calc.launch_count()
    calc.do_convolution(T(do.ptr, abi.FP32, xs, mem_space=1), *tens, cp, abi.OP_DEDX)
    assert calc.launch_count() - before == 4
    calc.do_convolution(T(do16.ptr, abi.BF16, xs, mem_space=1), *tens, cp, abi.OP_DEDX, abi.RM_NE, abi.make_cast_params(abi.RM_NE))
    calc.sync(20_000_000_000)
    out, out16 = do.download(np.float32), do16.download(np.uint16)
    img_x, img_y = int(np.prod(xs[:3])), int(np.prod(ys[:3]))
    xs1, ys1 = xs[:3] + [1], ys[:3] + [1]
    for img in (0, xs[3] - 1):
        yi = yb[img * img_y:(img + 1) * img_y]
        xi = xb[img * img_x:(img + 1) * img_x]
        r = np.zeros(img_x, np.float32)
        assert best_oracle.conv(T(r, abi.FP32, xs1), T(xi, abi.BF16, xs1), T(wb, abi.BF16, ws), T(yi, abi.BF16, ys1), cp, abi.OP_DEDX) == 0
        sabs = util.conv_sum_abs(best_oracle, (xs1, ws, ys1), (xi, wb, yi), abi.BF16, cp, abi.OP_DEDX)
        got = out[img * img_x:(img + 1) * img_x]
        util.assert_acc(got, r, sabs, "stride-2 dedx image %d" % img)
        got16, ref16 = out16[img * img_x:(img + 1) * img_x], port.fp32_to_bf16(r)
        inexact, far = util.check_rounded(got16, ref16, 16, util.bf16_to_f32(got16), util.bf16_to_f32(ref16), sabs, "stride-2 dedx bf16 image %d" % img)
        assert inexact <= 0.02 * img_x
    for b in (dx, dw, dy, do, do16):
        b.free()


def test_batched_attention_gemm(calc, best_oracle, port):
    """The attention-shaped batch: 64 x ([4096 x 128] . [128 x 4096]^T-style abt) fp8_143 -> bf16. K = 128 sums of fp8
    products are exact in fp32, so rounded outputs are compared bit for bit on sampled batches."""
    wl = bench.WORKLOADS["fp8_bgemm_attn"]
    B, M, N, K = 64, 4096, 4096, 128
    xb, wb = bench.synth_inputs(wl, seed=5)
    kw = dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL)
    dx, dw, do = calc.to_device(xb), calc.to_device(wb), calc.alloc(B * M * N * 2)
    calc.do_batch_gemm(T(do.ptr, abi.BF16, [N, M, B], mem_space=1), T(dx.ptr, abi.FP8_143, [K, M, B], mem_space=1, **kw),
                       T(dw.ptr, abi.FP8_143, [K, N, B], mem_space=1, **kw), abi.OP_ABT, abi.make_cast_params(abi.RM_NE))
    calc.sync(20_000_000_000)
    out = do.download(np.uint16).reshape(B, M, N)
    rows = 64
    for b in (0, 37, 63):
        xa = np.ascontiguousarray(xb.reshape(B, M, K)[b, 1000:1000 + rows])
        wa = np.ascontiguousarray(wb.reshape(B, N, K)[b])
        acc = np.zeros(rows * N, np.float32)
        assert best_oracle.bgemm(T(acc, abi.FP32, [N, rows]), T(xa, abi.FP8_143, [K, rows], **kw), T(wa, abi.FP8_143, [K, N], **kw), abi.OP_ABT) == 0
        ref = port.fp32_to_bf16(acc).reshape(rows, N)
        assert (out[b, 1000:1000 + rows] == ref).mean() > 0.999
        sabs = util.sum_abs_products(util.decode(xa, abi.FP8_143, 7, 2, port).reshape(rows, K), util.decode(wa, abi.FP8_143, 7, 2, port).reshape(N, K).T)
        util.check_rounded(out[b, 1000:1000 + rows], ref, 16, util.bf16_to_f32(out[b, 1000:1000 + rows]), util.bf16_to_f32(ref), sabs, "batched K=128")
    for buf in (dx, dw, do):
        buf.free()


def test_mixed_fp8_mlp_projection(calc, best_oracle, port):
    """The MLP projection: fp8_152 activations [16384 x 8192] times fp8_143 weights [8192 x 28672] -> bf16."""
    wl = bench.WORKLOADS["fp8_mlp"]
    M, N, K = wl["M"], wl["N"], wl["K"]
    xb, wb = bench.synth_inputs(wl, seed=6)
    kx, kw_ = dict(fp_bias=15, inf_nan_mode=abi.INFNAN_FULL), dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL)
    dx, dw, do = calc.to_device(xb), calc.to_device(wb), calc.alloc(M * N * 2)
    calc.do_batch_gemm(T(do.ptr, abi.BF16, [N, M], mem_space=1), T(dx.ptr, abi.FP8_152, [K, M], mem_space=1, **kx),
                       T(dw.ptr, abi.FP8_143, [N, K], mem_space=1, **kw_), abi.OP_AB, abi.make_cast_params(abi.RM_NE))
    calc.sync(30_000_000_000)
    rows = 8
    pick = np.array([0, 1, 4095, 4096, 9999, 12345, 16382, 16383])
    out = np.empty((rows, N), np.uint16)
    full = do.download(np.uint16).reshape(M, N)
    out[:] = full[pick]
    del full
    xa = np.ascontiguousarray(xb.reshape(M, K)[pick])
    acc = np.zeros(rows * N, np.float32)
    assert best_oracle.bgemm(T(acc, abi.FP32, [N, rows]), T(xa, abi.FP8_152, [K, rows], **kx), T(wb, abi.FP8_143, [N, K], **kw_), abi.OP_AB) == 0
    ref = port.fp32_to_bf16(acc).reshape(rows, N)
    sabs = util.sum_abs_products(util.decode(xa, abi.FP8_152, 15, 0, port).reshape(rows, K), util.decode(wb, abi.FP8_143, 7, 2, port).reshape(K, N))
    inexact, far = util.check_rounded(out, ref, 16, util.bf16_to_f32(out), util.bf16_to_f32(ref), sabs, "fp8 MLP")
    assert inexact <= 0.01 * rows * N
    for buf in (dx, dw, do):
        buf.free()


def test_full_size_properties_fp8_gemm(calc):
    """Size-independent properties at the full 8192^3 size: exact linearity under power-of-two scaling
    (bias 7 vs bias 11 operands hold the same codes: outputs differ by exactly 2^-4 per operand), row
    permutation invariance, and identity weights reproduce the input."""
    n = 8192
    wl = bench.WORKLOADS["fp8_gemm_8192"]
    xb, wb = bench.synth_inputs(wl, seed=9)
    dx, dw = calc.to_device(xb), calc.to_device(wb)
    d1, d2 = calc.alloc(n * n * 4), calc.alloc(n * n * 4)

    def gemm(dst, x_ptr, w_ptr, bx, bw):
        calc.do_batch_gemm(T(dst.ptr, abi.FP32, [n, n], mem_space=1), T(x_ptr, abi.FP8_143, [n, n], mem_space=1, fp_bias=bx, inf_nan_mode=2),
                           T(w_ptr, abi.FP8_143, [n, n], mem_space=1, fp_bias=bw, inf_nan_mode=2), abi.OP_AB)
    gemm(d1, dx.ptr, dw.ptr, 7, 7)
    gemm(d2, dx.ptr, dw.ptr, 11, 7)
    calc.sync(20_000_000_000)
    a, b = d1.download(np.float32), d2.download(np.float32)
    assert (a == b * np.float32(16.0)).all()          # the bias fold is an exact power-of-two scale
    # permuting rows of A permutes rows of C, bit for bit
    perm = np.random.default_rng(1).permutation(n)
    dxp = calc.to_device(np.ascontiguousarray(xb.reshape(n, n)[perm]))
    gemm(d2, dxp.ptr, dw.ptr, 7, 7)
    calc.sync(20_000_000_000)
    assert (d2.download(np.float32).reshape(n, n).view(np.uint32) == a.reshape(n, n)[perm].view(np.uint32)).all()
    # identity weights (1.0 = code 0x38 at bias 7): C == decode(A) exactly
    eye = np.zeros((n, n), np.uint8)
    np.fill_diagonal(eye, 0x38)
    de = calc.to_device(eye)
    gemm(d2, dx.ptr, de.ptr, 7, 7)
    calc.sync(20_000_000_000)
    from oracle import Port
    assert (d2.download(np.float32) == Port().fp8_to_fp32(xb, 4, 7, 2)).all()
    for buf in (dx, dw, d1, d2, dxp, de):
        buf.free()


def _exact_calculator():
    import intel_gaudi3_software_b200 as pkg
    c = pkg.Calculator(device=0)
    c.set_accumulation(abi.ACC_CHIP_EXACT)
    return c


def test_fp8_gemm_8192_every_output_against_the_exact_mode(calc):
    """The fp8 8192^3 GEMM, all 67 M outputs: the tensor-core accumulators against the bit-exact Gaudi3 mode (itself pinned to
    the reference on the smaller cases and the committed golden outputs), within 1e-5 * sum|a_k b_k| per element; and the bf16
    outputs of the two under the reference's own comparator rule, on the device."""
    wl = bench.WORKLOADS["fp8_gemm_8192"]
    n = 8192
    xb, wb = bench.synth_inputs(wl, seed=2)
    kw = dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL, mem_space=1)
    ex = _exact_calculator()
    dx, dw = calc.to_device(xb), calc.to_device(wb)
    d_fast, d_exact, d_abs = calc.alloc(n * n * 4), calc.alloc(n * n * 4), calc.alloc(n * n * 4)
    x, w = T(dx.ptr, abi.FP8_143, [n, n], **kw), T(dw.ptr, abi.FP8_143, [n, n], **kw)
    calc.do_batch_gemm(T(d_fast.ptr, abi.FP32, [n, n], mem_space=1), x, w, abi.OP_AB)
    calc.sync(20_000_000_000)
    ex.do_batch_gemm(T(d_exact.ptr, abi.FP32, [n, n], mem_space=1), x, w, abi.OP_AB)
    ex.sync(60_000_000_000)
    # sum|a||b| with the sign bits cleared, on the tensor cores (exact enough for a bound)
    dxa, dwa = calc.to_device(xb & 0x7F), calc.to_device(wb & 0x7F)
    calc.do_batch_gemm(T(d_abs.ptr, abi.FP32, [n, n], mem_space=1), T(dxa.ptr, abi.FP8_143, [n, n], **kw), T(dwa.ptr, abi.FP8_143, [n, n], **kw), abi.OP_AB)
    calc.sync(20_000_000_000)
    fast, exact, sabs = d_fast.download(np.float32), d_exact.download(np.float32), d_abs.download(np.float32)
    worst = 0.0
    for lo in range(0, n * n, 1 << 24):   # in slabs, to keep host memory modest
        hi = lo + (1 << 24)
        d = np.abs(fast[lo:hi].astype(np.float64) - exact[lo:hi])
        worst = max(worst, float((d / np.maximum(sabs[lo:hi], 1e-30)).max()))
    assert worst <= util.ACC_TOL, worst
    # bf16 outputs: fused cast on the tensor-core path against exact accumulators cast separately
    o_fast, o_exact = calc.alloc(n * n * 2), calc.alloc(n * n * 2)
    cp = abi.make_cast_params(abi.RM_NE)
    calc.do_batch_gemm(T(o_fast.ptr, abi.BF16, [n, n], mem_space=1), x, w, abi.OP_AB, cp)
    calc.sync(20_000_000_000)
    ex.do_activation(T(o_exact.ptr, abi.BF16, [n * n], mem_space=1), T(d_exact.ptr, abi.FP32, [n * n], mem_space=1), cp)
    ex.sync(20_000_000_000)
    bad, first = calc.compare(T(o_fast.ptr, abi.BF16, [n * n], mem_space=1), T(o_exact.ptr, abi.BF16, [n * n], mem_space=1), n)
    # The comparator allows 10 % (or 4 ulp): only outputs where the products cancel almost completely can differ by more while
    # the accumulators agree to 1e-5 * sum|ab| -- a handful in 67 M, each with |acc| far below sum|ab|.
    assert bad <= n * n // 1_000_000, (bad, first)
    if bad:
        assert abs(float(exact[first])) <= 1e-4 * float(sabs[first]), (first, float(exact[first]), float(sabs[first]))
    for b in (dx, dw, dxa, dwa, d_fast, d_exact, d_abs, o_fast, o_exact):
        b.free()
    ex.close()


@pytest.mark.parametrize("opname", ["conv_fwd", "conv_dedx", "conv_dedw"])
def test_resnet_conv_every_output_against_the_exact_mode(calc, opname):
    """The ResNet-shaped convolutions at full size: implicit-GEMM convolutions on the tensor cores against the bit-exact mode (im2col + exact GEMM
    + col2im, the reference's own lowering), all outputs, |fast - exact| <= 1e-5 * sum|a_k b_k| per element (dedw's 200704-term sums
    included: the chip truncates after every block of eight, which biases its sums toward zero, inside the same bound)."""
    wl = bench.WORKLOADS[opname]
    xs, ws, ys = bench.conv_shapes()
    xb, wb, yb = bench.synth_inputs(wl, seed=3)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    op = wl["op"]
    oshape = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[op]
    n_out = int(np.prod(oshape))
    ex = _exact_calculator()
    dx, dw, dy = calc.to_device(xb), calc.to_device(wb), calc.to_device(yb)
    d_fast, d_exact = calc.alloc(n_out * 4), calc.alloc(n_out * 4)
    tens = (T(dx.ptr, abi.BF16, xs, mem_space=1), T(dw.ptr, abi.BF16, ws, mem_space=1), T(dy.ptr, abi.BF16, ys, mem_space=1))
    calc.do_convolution(T(d_fast.ptr, abi.FP32, oshape, mem_space=1), *tens, cp, op)
    calc.sync(20_000_000_000)
    ex.do_convolution(T(d_exact.ptr, abi.FP32, oshape, mem_space=1), *tens, cp, op)
    ex.sync(120_000_000_000)
    fast, exact = d_fast.download(np.float32), d_exact.download(np.float32)
    assert np.isfinite(exact).all() and np.abs(exact).max() > 0
    # sum|a_k b_k| per output: the same convolution on the operands' absolute values, on the tensor cores (exact enough for a bound)
    da = [calc.to_device(util.clear_signs(b, abi.BF16)) for b in (xb, wb, yb)]
    d_abs = calc.alloc(n_out * 4)
    calc.do_convolution(T(d_abs.ptr, abi.FP32, oshape, mem_space=1), T(da[0].ptr, abi.BF16, xs, mem_space=1), T(da[1].ptr, abi.BF16, ws, mem_space=1),
                        T(da[2].ptr, abi.BF16, ys, mem_space=1), cp, op)
    calc.sync(20_000_000_000)
    sabs = d_abs.download(np.float32)
    util.assert_acc(fast, exact, sabs, opname + " against the exact mode")
    for b in da + [d_abs]:
        b.free()
    for b in (dx, dw, dy, d_fast, d_exact):
        b.free()
    ex.close()
