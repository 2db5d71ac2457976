"""The allocation-free split-K GEMM (mmeb200_gemm_splitk_static).

Who needs it: callers that are not allowed to allocate device memory at the moment they need a GEMM --
a plug-in running under a framework's memory pool that was handed exactly its input and output
buffers, a latency-critical loop that must stay clear of the allocator's lock, a service whose
device-memory budget was fixed when it started. The entry point keeps the fp32 partial sums of the
split reduction in a fixed 16 MiB array that is part of the library image, and calls no allocator.

The test calls it through the C ABI on device-resident tensors and compares with the ordinary entry
point (mmeb200_bgemm) and with the CPU oracle on the same inputs, twice in a row with different shapes,
so that partial sums left behind by the first call would show up in the second. It also checks the
property the entry point exists for: after a warm-up call (the one-time set-up) free device memory is
the same before and after a call. This file sorts last on purpose: a run that stops at the first
failure has then already run every other test.
"""
import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
import util

pytestmark = pytest.mark.gpu


def run_both(calc, rng, M, N, K, op, splits, dtype=abi.BF16, oracle=None, port=None):
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
    calc.sync()
    free_before = calc.mem_info()[0]
    calc.gemm_splitk_static(T(d_static.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE), x, w, op, splits)
    calc.sync()
    free_after = calc.mem_info()[0]
    calc.do_batch_gemm(T(d_plain.ptr, abi.FP32, [N, M], mem_space=abi.MEM_DEVICE), x, w, op)
    calc.sync(10_000_000_000)
    a, b = d_static.download(np.float32), d_plain.download(np.float32)
    for buf in (dx, dw, d_static, d_plain):
        buf.free()
    # same products, different summation order: the accumulator tolerance of the other GPU tests
    assert np.abs(a.astype(np.float64) - b.astype(np.float64)).max() <= util.ACC_TOL * bound, (M, N, K, op, splits)
    if oracle is not None:
        # against the CPU oracle, per element: |gpu - ref| <= 1e-5 * sum|a_k b_k|
        ref = np.zeros(M * N, np.float32)
        assert oracle.bgemm(T(ref, abi.FP32, [N, M]), T(xb, dtype, xs, **kw), T(wb, dtype, ws, **kw), op) == 0
        xf = util.decode(xb, dtype, 7, 2, port).reshape(xs[::-1])
        wf = util.decode(wb, dtype, 7, 2, port).reshape(ws[::-1])
        sabs = util.sum_abs_products(xf.T if tA else xf, wf.T if tB else wf)
        util.assert_acc(a, ref, sabs, "allocation-free gemm %dx%dx%d" % (M, N, K))
    return a, free_before, free_after


def test_two_calls_in_a_row_match_the_ordinary_entry_point(best_oracle, port):
    calc = pkg.Calculator(device=0)
    rng = np.random.default_rng(2024)
    first, _, _ = run_both(calc, rng, 256, 384, 2048, abi.OP_AB, 4, oracle=best_oracle, port=port)
    # second call: smaller output, more splits, other orientation -- reads only what it wrote itself
    second, before, after = run_both(calc, rng, 100, 72, 4096, abi.OP_ABT, 16, oracle=best_oracle, port=port)
    assert np.isfinite(first).all() and np.isfinite(second).all()
    # the first call was the warm-up (one-time set-up); from then on a call leaves free device memory as it found it
    assert before == after, (before, after)
    _, before, after = run_both(calc, rng, 128, 128, 1024, abi.OP_AB, 8, dtype=abi.FP8_143, oracle=best_oracle, port=port)
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
