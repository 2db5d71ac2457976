"""The fused dedw exchange (split-K reduction + reduce-scatter to the owner ranks + rank-ordered sum + all-gather, all over
plain peer stores).

One GPU: a group of world 1 runs the same kernels (scatter into its own slot, flags, bounded waits, owner sum, copy)
and must reproduce plain dedw bit for bit, in the tensor-core mode and in the bit-exact accumulation mode. Two or more GPUs: one process per GPU over real peer memory
(skipped where fewer GPUs are visible). A wait that cannot be satisfied (a flag nobody sets) must end by
itself with MMEB200_ERR_DEVICE_WAIT and leave the context usable -- no GPU fault is involved."""
import os
import subprocess
import sys

import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
from intel_gaudi3_software_b200.multi_gpu import PeerExchange
import util

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CASE = dict(xs=[64, 32, 32, 4], ws=[64, 64, 3, 3], ys=[64, 32, 32, 4])


def inputs(seed):
    rng = np.random.default_rng(seed)
    xb = util.gen_bf16(rng, int(np.prod(CASE["xs"])), "normal")
    yb = util.gen_bf16(rng, int(np.prod(CASE["ys"])), "normal", 0.01)
    wb = np.zeros(int(np.prod(CASE["ws"])), np.uint16)
    return xb, wb, yb


def test_world_of_one_matches_plain_dedw(calc):
    xb, wb, yb = inputs(0)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    x, w, y = T(xb, abi.BF16, CASE["xs"]), T(wb, abi.BF16, CASE["ws"]), T(yb, abi.BF16, CASE["ys"])
    n = int(np.prod(CASE["ws"]))
    plain = np.zeros(n, np.float32)
    calc.do_convolution(T(plain, abi.FP32, CASE["ws"]), x, w, y, cp, abi.OP_DEDW)
    ex = PeerExchange(calc, n)
    for it in range(5):  # both buffer sets, several steps each
        fused = np.full(n, 9.0, np.float32)
        ex.dedw_allreduce(T(fused, abi.FP32, CASE["ws"]), x, w, y, cp)
        assert (fused.view(np.uint32) == plain.view(np.uint32)).all(), it
    ex.close()


def test_world_of_one_in_the_exact_accumulation_mode():
    """The bit-exact mode takes the general lowering (im2col + exact GEMM); its partial dW must go through the same exchange."""
    c = pkg.Calculator(device=0, accumulation=abi.ACC_CHIP_EXACT)
    xb, wb, yb = inputs(3)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    x, w, y = T(xb, abi.BF16, CASE["xs"]), T(wb, abi.BF16, CASE["ws"]), T(yb, abi.BF16, CASE["ys"])
    n = int(np.prod(CASE["ws"]))
    plain = np.zeros(n, np.float32)
    c.do_convolution(T(plain, abi.FP32, CASE["ws"]), x, w, y, cp, abi.OP_DEDW)
    ex = PeerExchange(c, n)
    for it in range(3):
        fused = np.full(n, 9.0, np.float32)
        ex.dedw_allreduce(T(fused, abi.FP32, CASE["ws"]), x, w, y, cp)
        assert (fused.view(np.uint32) == plain.view(np.uint32)).all(), it
    ex.close()
    c.close()


def test_world_of_one_deferred_output_on_device_tensors(calc):
    """Device tensors with the deferred output: the final add runs on a side stream and is joined by sync()."""
    xb, wb, yb = inputs(2)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    n = int(np.prod(CASE["ws"]))
    plain = np.zeros(n, np.float32)
    calc.do_convolution(T(plain, abi.FP32, CASE["ws"]), T(xb, abi.BF16, CASE["xs"]), T(wb, abi.BF16, CASE["ws"]), T(yb, abi.BF16, CASE["ys"]), cp, abi.OP_DEDW)
    ex = PeerExchange(calc, n, deferred_output=True)
    dx, dw, dy, dout = calc.to_device(xb), calc.to_device(wb), calc.to_device(yb), calc.alloc(n * 4)
    dev = abi.MEM_DEVICE
    for it in range(5):
        ex.dedw_allreduce(T(dout.ptr, abi.FP32, CASE["ws"], mem_space=dev), T(dx.ptr, abi.BF16, CASE["xs"], mem_space=dev),
                          T(dw.ptr, abi.BF16, CASE["ws"], mem_space=dev), T(dy.ptr, abi.BF16, CASE["ys"], mem_space=dev), cp)
    calc.sync(10_000_000_000)
    assert (dout.download(np.float32).view(np.uint32) == plain.view(np.uint32)).all()
    ex.close()
    for b in (dx, dw, dy, dout):
        b.free()


def test_unsatisfiable_wait_ends_by_itself():
    c = pkg.Calculator(device=0)
    xb, wb, yb = inputs(1)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    x, w, y = T(xb, abi.BF16, CASE["xs"]), T(wb, abi.BF16, CASE["ws"]), T(yb, abi.BF16, CASE["ys"])
    n = int(np.prod(CASE["ws"]))
    ex = PeerExchange(c, n)
    g = ex.groups[0]
    g.step = 3   # pretends three exchanges happened: the flag can never reach the target
    out = np.zeros(n, np.float32)
    with pytest.raises(pkg.MmeError) as ei:
        c.do_convolution_dedw_allreduce(T(out, abi.FP32, CASE["ws"]), x, w, y, cp, g)
    assert ei.value.status == abi.ERR_DEVICE_WAIT
    # the context still works
    plain = np.zeros(n, np.float32)
    c.do_convolution(T(plain, abi.FP32, CASE["ws"]), x, w, y, cp, abi.OP_DEDW)
    assert np.isfinite(plain).all() and np.abs(plain).max() > 0
    c.close()


def test_two_ranks_over_peer_memory():
    lib = abi.load_library()
    if lib.mmeb200_device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    p = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", "29577", os.path.join(ROOT, "tests", "peer_exchange_worker.py")], capture_output=True, text=True,
                       timeout=600, env=env)
    assert p.returncode == 0, p.stdout[-3000:] + p.stderr[-3000:]
    assert "PEER EXCHANGE OK" in p.stdout
