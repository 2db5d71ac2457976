"""The benchmark configurations of the MME path and their seeded synthetic inputs.

No public data set is involved in this path: the configurations are shapes, data types and value
distributions, and these generators are the workload. They are shared by the benchmark, the
multi-GPU driver and the parity tests, so that every side of a comparison is fed the same bytes.

FLOPs of a step = 2*M*N*K (a convolution counts as its implicit GEMM); algorithmic bytes = every
operand read once + the output written once in its final type.
"""
import numpy as np

from . import abi

L2_BYTES = 126 * 1024 * 1024

# name -> description of one step.
WORKLOADS = {
    # fp8_143 (E4M3) GEMM 8192^3 -> bf16, round to nearest even; exponent bias 7, then 11 (the bias fold)
    "fp8_gemm_8192": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                          out_dtype=abi.BF16, bound="tensor", peak="fp8", dtype="fp8_143"),
    "fp8_gemm_8192_bias11": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=11,
                                 out_dtype=abi.BF16, bound="tensor", peak="fp8", dtype="fp8_143"),
    # the same GEMM with the seeded stochastic-rounding cast (counter-based stream, fused into the epilogue)
    "fp8_gemm_8192_sr": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                             out_dtype=abi.BF16, bound="tensor", peak="fp8", dtype="fp8_143", stochastic=True),
    # ... with fp8_143 output: round-to-nearest-even + clipping (hardware conversion), and stochastic rounding. The operands
    # carry exponent bias 15 (a per-tensor scale of 2^-8 each), which puts the products' sums (sigma about 14) inside the
    # output format's range; with bias 7 nearly every output would overflow and be clipped.
    "fp8_gemm_8192_fp8out": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=15,
                                 out_dtype=abi.FP8_143, bound="tensor", peak="fp8", dtype="fp8_143", clip=True),
    "fp8_gemm_8192_fp8out_sr": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=15,
                                    out_dtype=abi.FP8_143, bound="tensor", peak="fp8", dtype="fp8_143", stochastic=True),
    "bf16_gemm_8192": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.BF16, w_dtype=abi.BF16, bias=0,
                           out_dtype=abi.BF16, bound="tensor", peak="bf16", dtype="bf16"),
    # bf16 1024^3 -> fp32: the case the reference's CPU calculator runs in full
    "bf16_gemm_1024": dict(kind="gemm", M=1024, N=1024, K=1024, in_dtype=abi.BF16, w_dtype=abi.BF16, bias=0,
                           out_dtype=abi.FP32, bound="tensor", peak="bf16", dtype="bf16"),
    # fp32 and tf32 operands (three tf32 products per fp32 pair; tf32 operands are rounded first)
    "fp32_gemm_4096": dict(kind="gemm", M=4096, N=4096, K=4096, in_dtype=abi.FP32, w_dtype=abi.FP32, bias=0,
                           out_dtype=abi.FP32, bound="tensor", peak="tf32x3", dtype="fp32"),
    "tf32_gemm_4096": dict(kind="gemm", M=4096, N=4096, K=4096, in_dtype=abi.TF32, w_dtype=abi.TF32, bias=0,
                           out_dtype=abi.FP32, bound="tensor", peak="tf32", dtype="tf32"),
    # attention-shaped batch: 64 x ([4096 x 128] . [4096 x 128]^T), HBM-bound by its bf16 output
    "fp8_bgemm_attn": dict(kind="gemm", M=4096, N=4096, K=128, batch=64, op=abi.OP_ABT, in_dtype=abi.FP8_143,
                           w_dtype=abi.FP8_143, bias=7, out_dtype=abi.BF16, bound="hbm", peak="fp8", dtype="fp8_143"),
    # MLP projection: fp8_152 activations x fp8_143 weights
    "fp8_mlp": dict(kind="gemm", M=16384, N=28672, K=8192, in_dtype=abi.FP8_152, w_dtype=abi.FP8_143, bias=7,
                    out_dtype=abi.BF16, bound="tensor", peak="fp8", dtype="fp8_152xfp8_143"),
    # the optional bit-exact Gaudi3 accumulation (integer emulation on the CUDA cores; no tensor cores)
    "fp8_gemm_2048_exact": dict(kind="gemm", M=2048, N=2048, K=2048, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                                out_dtype=abi.FP32, bound="tensor", peak="fp8", dtype="fp8_143", exact=True),
    # ResNet-shaped 3x3 convolution, NHWC 64 x 56 x 56 x 256 -> 256, stride 1, pad 1
    "conv_fwd": dict(kind="conv", op=abi.OP_FWD, out_dtype=abi.BF16, bound="tensor", peak="bf16", dtype="bf16"),
    "conv_dedx": dict(kind="conv", op=abi.OP_DEDX, out_dtype=abi.BF16, bound="tensor", peak="bf16", dtype="bf16"),
    "conv_dedw": dict(kind="conv", op=abi.OP_DEDW, out_dtype=abi.FP32, bound="tensor", peak="bf16", dtype="bf16"),
    # same dedw, the cross-GPU sum fused into the split-K reduction (peer stores, owner sums, peer stores back)
    "conv_dedw_fused": dict(kind="conv", op=abi.OP_DEDW, out_dtype=abi.FP32, bound="tensor", peak="bf16", dtype="bf16",
                            fused_exchange=True),
    # the same convolution with stride 2 (dedx of a strided convolution)
    "conv_dedx_stride2": dict(kind="conv", op=abi.OP_DEDX, out_dtype=abi.BF16, bound="tensor", peak="bf16", dtype="bf16",
                              stride=2),
}
# HBM-bound helper kernels of the path (cast, comparator, memory-write reduction, tensor generator): one pass over n
# elements. value = algorithmic GB/s (bytes each kernel must read and write once); the tensors are far larger than L2.
STREAM_WORKLOADS = {
    "cast_f32_to_bf16": dict(kind="stream", n=1 << 28, bytes_per_elem=6, dtype="f32"),          # doActivation, RNE
    "cast_f32_to_fp8": dict(kind="stream", n=1 << 28, bytes_per_elem=5, dtype="f32"),           # doActivation, fp8_143 RNE + clip
    "cast_f32_to_bf16_sr": dict(kind="stream", n=1 << 28, bytes_per_elem=6, dtype="f32"),       # doActivation, stochastic (Philox)
    "compare_bf16": dict(kind="stream", n=1 << 29, bytes_per_elem=4, dtype="bf16"),             # TensorComparator rule
    "memory_write_add_f32": dict(kind="stream", n=1 << 28, bytes_per_elem=12, dtype="f32"),     # doMemoryWrite add: 2 reads + 1 write
    "generate_uniform_bf16": dict(kind="stream", n=1 << 29, bytes_per_elem=2, dtype="bf16"),    # RandomSimTensorGenerator
}
WORKLOADS.update(STREAM_WORKLOADS)
CONV = dict(C=256, K=256, W=56, H=56, B=64, S=3, R=3, pad=1)


def bf16_to_f32(u16):
    return (np.asarray(u16, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_rne(x):
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs; same result as the reference's fp32_to_bf16 RNE)."""
    b = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    return ((b + 0x7FFF + ((b >> 16) & 1)) >> 16).astype(np.uint16)


def quantise_fp8(v, dtype, bias):
    """RNE cast of N(0,1) draws, scaled to amax = max finite, to fp8 code bytes (numpy, vectorised).

    1-4-3 uses the 'minimal Inf/NaN' convention (max 448 * 2^(7-bias)); 1-5-2 the full one (max 57344 * 2^(15-bias)).
    The tensor's bias only rescales the values, so the codes do not depend on it.
    """
    man = 3 if dtype == abi.FP8_143 else 2
    hw_bias = 7 if dtype == abi.FP8_143 else 15
    maxv = (448.0 if dtype == abi.FP8_143 else 57344.0)
    a = v * np.float32(maxv / np.abs(v).max())          # in hardware-bias units
    sign = (a < 0).astype(np.uint8) << 7
    m = np.abs(a).astype(np.float32)
    e = np.frexp(m)[1].astype(np.int32) - 1           # m = f * 2^(e+1), f in [0.5, 1)
    e = np.maximum(e, 1 - hw_bias)                       # denormal range shares the smallest exponent
    q = np.rint(m / np.exp2(e - man).astype(np.float32)).astype(np.int32)   # rint = round half to even
    over = q >= (2 << man)
    e = np.where(over, e + 1, e)
    q = np.where(over, q >> 1, q)
    code = np.where(q < (1 << man), q, ((e + hw_bias) << man) | (q & ((1 << man) - 1))).astype(np.uint8)
    return (code | sign).astype(np.uint8)


def conv_shapes(wl=None, images=None):
    """(x, w, y) sizes in the reference's convention (fastest dimension first) of the convolution workloads."""
    c = CONV
    s = (wl or {}).get("stride", 1)
    b = c["B"] if images is None else images
    wo = (c["W"] + 2 * c["pad"] - c["S"]) // s + 1
    ho = (c["H"] + 2 * c["pad"] - c["R"]) // s + 1
    return [c["C"], c["W"], c["H"], b], [c["K"], c["C"], c["S"], c["R"]], [c["K"], wo, ho, b]


def workload_counts(wl, rows=None, images=None):
    """(flops, algorithmic bytes) of one step; `rows` / `images` restrict a GEMM / convolution to a shard."""
    if wl["kind"] == "gemm":
        b = wl.get("batch", 1)
        M, N, K = (wl["M"] if rows is None else rows), wl["N"], wl["K"]
        flops = 2.0 * M * N * K * b
        byts = b * (M * K * abi.ELEM_SIZE[wl["in_dtype"]] + K * N * abi.ELEM_SIZE[wl["w_dtype"]] +
                    M * N * abi.ELEM_SIZE[wl["out_dtype"]])
        return flops, float(byts)
    xs, ws, ys = conv_shapes(wl, images)
    pixels = ys[1] * ys[2] * ys[3]
    flops = 2.0 * pixels * ws[0] * ws[1] * ws[2] * ws[3]
    nx, nw, ny = int(np.prod(xs)), int(np.prod(ws)), int(np.prod(ys))
    if wl["op"] == abi.OP_FWD:
        byts = 2 * nx + 2 * nw + abi.ELEM_SIZE[wl["out_dtype"]] * ny
    elif wl["op"] == abi.OP_DEDX:
        byts = 2 * ny + 2 * nw + abi.ELEM_SIZE[wl["out_dtype"]] * nx
    else:
        byts = 2 * nx + 2 * ny + abi.ELEM_SIZE[wl["out_dtype"]] * nw
    return flops, float(byts)


def operand_biases(wl):
    """(bias of x, bias of w) of a GEMM workload's fp8 operands."""
    x_bias = wl["bias"] if wl["in_dtype"] == abi.FP8_143 else 15
    w_bias = 7 if wl["in_dtype"] != abi.FP8_143 else wl["bias"]
    return x_bias, w_bias


def inf_nan_mode(dtype):
    return abi.INFNAN_MINIMAL if dtype == abi.FP8_143 else abi.INFNAN_FULL


def synth_inputs(wl, seed, rows=None, images=None):
    """Seeded synthetic operands with the configuration's shapes and value distributions.

    GEMM: (x, w). bf16 operands are uniform[-1, 1] rounded to nearest even; fp32 / tf32 operands uniform[-1, 1];
    fp8 operands are N(0,1) scaled per tensor to amax = the format's largest finite value, RNE-cast, generated as code
    bytes through a numpy quantiser that reproduces the reference's RNE cast for in-range values.
    Convolution: (x, w, y): activations N(0,1), weights Kaiming-normal, output gradient N(0, 0.01), all bf16.
    `rows` / `images` generate a shard of that many rows of A / images.
    """
    rng = np.random.default_rng(seed)
    if wl["kind"] == "gemm":
        b = wl.get("batch", 1)
        M = rows if rows is not None else wl["M"]
        N, K = wl["N"], wl["K"]

        def make(n, dtype, bias):
            if dtype == abi.BF16:
                return f32_to_bf16_rne(rng.uniform(-1, 1, n).astype(np.float32))
            if dtype in (abi.FP32, abi.TF32):
                return rng.uniform(-1, 1, n).astype(np.float32)
            return quantise_fp8(rng.standard_normal(n, dtype=np.float32), dtype, bias)
        xb, wb = operand_biases(wl)
        return make(M * K * b, wl["in_dtype"], xb), make(K * N * b, wl["w_dtype"], wb)
    xs, ws, ys = conv_shapes(wl, images)
    x = f32_to_bf16_rne(rng.standard_normal(int(np.prod(xs)), dtype=np.float32))
    w = f32_to_bf16_rne((rng.standard_normal(int(np.prod(ws)), dtype=np.float32) * np.float32(np.sqrt(2.0 / (ws[1] * ws[2] * ws[3])))))
    y = f32_to_bf16_rne((rng.standard_normal(int(np.prod(ys)), dtype=np.float32) * np.float32(0.01)))
    return x, w, y
