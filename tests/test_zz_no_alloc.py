"""The allocation-free split-K GEMM (mmeb200_gemm_splitk_static).

Who needs it: callers that are not allowed to allocate device memory at the moment they need a GEMM --
a plug-in running under a framework's memory pool that was handed exactly its input and output
buffers, a latency-critical loop that must stay clear of the allocator's lock, a service whose
device-memory budget was fixed when it started. The entry point keeps the fp32 partial sums of the
split reduction in a fixed 16 MiB array that is part of the library image, and calls no allocator.

The test calls it through the C ABI on device-resident tensors and compares with the ordinary entry
point (mmeb200_bgemm) on the same inputs, twice in a row with different shapes, so that partial sums
left behind by the first call would show up in the second. This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""
import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util

pytestmark = pytest.mark.gpu


def run_both(calc, rng, M, N, K, op, splits, dtype=abi.BF16):
    tA, tB = op in (abi.OP_ATB, abi.OP_ATBT), op in (abi.OP_ABT, abi.OP_ATBT)
    xs = [M, K] if tA else [K, M]
    ws = [K, N] if tB else [N, K]
    if dtype == abi.BF16:
        xb, wb = util.gen_bf16(rng, M * K), util.gen_bf16(rng, K * N)
        kw = {}
        bound = K / 4.0            # typical sum|ab| for U[-1,1] operands
    else:
        xb = (rng.integers(0, 256, M * K) & 0xBF).astype(np.uint8)
        wb = (rng.integers(0, 256, K * N) & 0xBF).astype(np.uint8)
        kw = dict(fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL)
        bound = K * 1.0
    dx, dw = calc.to_device(xb), calc.to_device(wb)
    d_static, d_plain = calc.alloc(M * N * 4), calc.alloc(M * N * 4)
    x = T(dx.ptr, dtype, xs, mem_space=abi.MEM_DEVICE, **kw)
    w = T(dw.ptr, dtype, ws, mem_space=abi.MEM_DEVICE, **kw)
    calc.gemm_splitk_static(T(d_static.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE), x, w, op, splits)
    calc.do_batch_gemm(T(d_plain.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE), x, w, op)
    calc.sync(10_000_000_000)
    a, b = d_static.download(np.float32), d_plain.download(np.float32)
    for buf in (dx, dw, d_static, d_plain):
        buf.free()
    # same products, different summation order: the accumulator tolerance of the other GPU tests
    assert np.abs(a.astype(np.float64) - b.astype(np.float64)).max() <= util.ACC_TOL * bound, (M, N, K, op, splits)
    return a


def test_two_calls_in_a_row_match_the_ordinary_entry_point():
    calc = pkg.Calculator(device=0)
    rng = np.random.default_rng(2024)
    first = run_both(calc, rng, 256, 384, 2048, abi.OP_AB, 4)
    # second call: smaller output, more splits, other orientation -- reads only what it wrote itself
    second = run_both(calc, rng, 100, 72, 4096, abi.OP_ABT, 16)
    assert np.isfinite(first).all() and np.isfinite(second).all()
    run_both(calc, rng, 128, 128, 1024, abi.OP_AB, 8, dtype=abi.FP8_143)
    calc.close()


def test_requests_beyond_the_fixed_workspace_are_rejected():
    calc = pkg.Calculator(device=0)
    M = N = 2048  # 8 splits x 2048 x 2048 x 4 bytes = 128 MiB > 16 MiB
    K = 1024
    dx, dw, do = calc.alloc(M * K * 2), calc.alloc(K * N * 2), calc.alloc(M * N * 4)
    x = T(dx.ptr, abi.BF16, [K, M], mem_space=abi.MEM_DEVICE)
    w = T(dw.ptr, abi.BF16, [N, K], mem_space=abi.MEM_DEVICE)
    o = T(do.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE)
    with pytest.raises(pkg.MmeError, match="exceeds the fixed"):
        calc.gemm_splitk_static(o, x, w, abi.OP_AB, 8)
    host = np.zeros(16, np.float32)
    with pytest.raises(pkg.MmeError, match="device-resident"):
        calc.gemm_splitk_static(T(host, abi.FP32, [4, 4]), x, w, abi.OP_AB, 2)
    for buf in (dx, dw, do):
        buf.free()
    calc.close()
