"""Generates tests/golden/golden_small.npz by running the UNMODIFIED reference calculator
(oracle/_ref/libmme_ref.so, built by oracle/Makefile from the reference checkout).

Run in a container that has the reference checkout:  python tests/golden/make_golden.py
The fixture pins the C restatement (tests/test_oracle_golden.py) and the GPU path
(tests/test_gpu_golden.py) where the reference itself is not available.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
from intel_gaudi3_software_b200 import abi  # noqa: E402
from intel_gaudi3_software_b200.abi import make_tensor as T  # noqa: E402
from oracle import Ref  # noqa: E402
import util  # noqa: E402

CONV_CASES = [
    # C, K, W, H, B, S, R, stride, pad, dil
    (8, 6, 7, 6, 2, 3, 3, (1, 1), (1, 1), (1, 1)),
    (5, 4, 9, 8, 2, 3, 2, (2, 1), (1, 0), (1, 2)),
    (16, 8, 6, 5, 1, 2, 3, (1, 2), (2, 1), (2, 1)),
]
GEMM_CASES = [
    # M, N, K, op, batch
    (1, 1, 5, abi.OP_AB, ()),
    (5, 5, 5, abi.OP_AB, ()),
    (13, 10, 21, abi.OP_AB, ()),
    (13, 10, 21, abi.OP_ABT, ()),
    (13, 10, 21, abi.OP_ATB, ()),
    (13, 10, 21, abi.OP_ATBT, ()),
    (24, 40, 72, abi.OP_AB, (3, 2)),
    (33, 17, 130, abi.OP_AB, ()),
]


def conv_shapes(c):
    C, K, W, H, B, S, R, st, pad, dil = c
    o = lambda i, k, s, p, d: (i + 2 * p - d * (k - 1) - 1) // s + 1  # noqa: E731
    return [C, W, H, B], [K, C, S, R], [K, o(W, S, st[0], pad[0], dil[0]), o(H, R, st[1], pad[1], dil[1]), B]


def main():
    r = Ref()
    rng = np.random.default_rng(20240607)
    out = {}
    # ---- conversions: every fp8 code, and a sample of fp32 inputs under every mode
    codes = np.arange(256, dtype=np.uint8)
    for ew, biases in ((4, (3, 7, 11, 15)), (5, (1, 15, 30))):
        for b in biases:
            for mode in (0, 1, 2):
                out["dec_%d_%d_%d" % (ew, b, mode)] = r.fp8_to_fp32(codes, ew, b, mode).view(np.uint32)
    n = 1200
    bits = rng.integers(0, 2**32, size=n, dtype=np.uint64).astype(np.uint32)
    ex = rng.integers(127 - 36, 127 + 18, size=n).astype(np.uint32)
    bits = np.concatenate([(bits & 0x807FFFFF) | (ex << 23), (bits & 0x80700000) | (ex << 23),
                           np.array([0, 0x80000000, 0x7F800000, 0xFF800000, 0x7FC00000, 0xFFC00001, 1, 0x80000001,
                                     0x007FFFFF, 0x7F7FFFFF, 0xFF7FFFFF], dtype=np.uint32)])
    lfsr = rng.integers(1, 2**32, size=bits.size, dtype=np.uint64).astype(np.uint32)
    out["cast_in"], out["cast_lfsr"] = bits, lfsr
    for rm in (0, 1, 2, 3, 4, 6, 7):
        out["bf16_rm%d" % rm] = r.fp32_to_bf16(bits, rm, lfsr, False, False, False)
        out["bf16_rm%d_clip_ftz" % rm] = r.fp32_to_bf16(bits, rm, lfsr, True, True, False)
        for ew, b, mode in ((4, 7, 2), (4, 11, 0), (4, 3, 1), (5, 15, 0), (5, 20, 2)):
            out["fp8_%d_%d_%d_rm%d" % (ew, b, mode, rm)] = r.fp32_to_fp8(bits, ew, b, rm, lfsr, False, False, False, False, mode)
            out["fp8_%d_%d_%d_rm%d_flags" % (ew, b, mode, rm)] = r.fp32_to_fp8(bits, ew, b, rm, lfsr, True, True, False, True, mode)
    # ---- GEMMs (bf16 operands) on the three chip models; fp8 and fp32-class operands on Gaudi3
    for i, (M, N, K, op, batch) in enumerate(GEMM_CASES):
        tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
        xs = ([M, K] if tA else [K, M]) + list(batch)
        ws = ([K, N] if tB else [N, K]) + list(batch)
        xb, wb = util.gen_bf16(rng, int(np.prod(xs))), util.gen_bf16(rng, int(np.prod(ws)))
        out["gemm%d_x" % i], out["gemm%d_w" % i] = xb, wb
        for chip in (0, 1, 2):
            o = np.zeros(M * N * int(np.prod(batch) if batch else 1), np.float32)
            assert r.bgemm(T(o, abi.FP32, [N, M] + list(batch)), T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), op, chip=chip) == 0
            out["gemm%d_chip%d" % (i, chip)] = o
    M, N, K = 16, 24, 40
    xb, wb = rng.integers(0, 256, M * K).astype(np.uint8), rng.integers(0, 256, K * N).astype(np.uint8)
    out["fp8gemm_x"], out["fp8gemm_w"] = xb, wb
    for j, (tx, tw, bx, bw, mx, mw) in enumerate(((9, 9, 7, 11, 2, 2), (10, 9, 15, 7, 0, 2), (9, 10, 3, 20, 1, 1), (9, 9, 15, 15, 0, 0))):
        o = np.zeros(M * N, np.float32)
        assert r.bgemm(T(o, abi.FP32, [N, M]), T(xb, tx, [K, M], fp_bias=bx, inf_nan_mode=mx),
                       T(wb, tw, [N, K], fp_bias=bw, inf_nan_mode=mw), abi.OP_AB) == 0
        out["fp8gemm_%d" % j] = o.view(np.uint32)
    xf, wf = rng.normal(0, 1, M * K).astype(np.float32), rng.normal(0, 1, K * N).astype(np.float32)
    out["f32gemm_x"], out["f32gemm_w"] = xf, wf
    for dt, nm in ((abi.FP32, "fp32"), (abi.TF32, "tf32")):
        o = np.zeros(M * N, np.float32)
        assert r.bgemm(T(o, abi.FP32, [N, M]), T(xf, dt, [K, M]), T(wf, dt, [N, K]), abi.OP_AB) == 0
        out["f32gemm_" + nm] = o
    # ---- convolutions (bf16) on Gaudi3
    for i, c in enumerate(CONV_CASES):
        xs, ws, ys = conv_shapes(c)
        cp = abi.make_conv_params(2, c[8], c[7], c[9])
        xb = util.gen_bf16(rng, int(np.prod(xs)), "normal")
        wb = util.gen_bf16(rng, int(np.prod(ws)), "normal", 0.1)
        yb = util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.01)
        out["conv%d_x" % i], out["conv%d_w" % i], out["conv%d_y" % i] = xb, wb, yb
        for op, shp, nm in ((abi.OP_FWD, ys, "fwd"), (abi.OP_DEDX, xs, "dedx"), (abi.OP_DEDW, ws, "dedw")):
            o = np.full(int(np.prod(shp)), 3.0, np.float32)
            assert r.conv(T(o, abi.FP32, shp), T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), T(yb, abi.BF16, ys), cp, op) == 0
            out["conv%d_%s" % (i, nm)] = o
    # ---- transposed_dedx: weights arrive as [C, K, S, R] with S mirrored (mme_reference_impl.cpp:625-647)
    c = CONV_CASES[0]
    xs, ws, ys = conv_shapes(c)
    cp = abi.make_conv_params(2, c[8], c[7], c[9])
    wt_shape = [ws[1], ws[0], ws[2], ws[3]]
    wtb = util.gen_bf16(rng, int(np.prod(wt_shape)), "normal", 0.1)
    o = np.zeros(int(np.prod(xs)), np.float32)
    assert r.conv(T(o, abi.FP32, xs), T(out["conv0_x"], abi.BF16, xs), T(wtb, abi.BF16, wt_shape), T(out["conv0_y"], abi.BF16, ys), cp,
                  abi.OP_TRANSPOSED_DEDX) == 0
    out["tdedx_w"], out["tdedx_out"] = wtb, o
    # ---- activation with the LFSR stream
    n = 700
    acc = (rng.normal(0, 1, n) * 10.0 ** rng.integers(-6, 6, n)).astype(np.float32)
    regs = rng.integers(1, 2**32, 256, dtype=np.uint64).astype(np.uint32)
    out["act_acc"], out["act_lfsr"] = acc, regs
    for od, bias, mode, nm in ((abi.BF16, 0, 0, "bf16"), (abi.FP8_143, 7, 2, "f143"), (abi.FP8_152, 15, 0, "f152")):
        for rm in (0, 4, 7):
            for relu in (0, 1):
                o = np.zeros(n, abi.NP_DTYPE[od])
                cp = abi.make_cast_params(rm, relu, clip_fp=(rm == 4))
                rc, _ = r.activation(T(o, od, [n], fp_bias=bias, inf_nan_mode=mode), T(acc.copy(), abi.FP32, [n]), cp, regs, 37)
                assert rc == 0
                out["act_%s_rm%d_relu%d" % (nm, rm, relu)] = o
    path = os.path.join(ROOT, "tests", "golden", "golden_small.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes,", len(out), "arrays")


if __name__ == "__main__":
    main()
