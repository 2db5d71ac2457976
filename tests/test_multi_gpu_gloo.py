"""The multi-GPU driver's host logic on CPU: world_size-2 gloo ranks plan their shards, run their
share through a stand-in calculator (the CPU oracle plays the GPU here -- test infrastructure only),
and the dedw partials are summed with a real torch.distributed all-reduce."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from intel_gaudi3_software_b200 import abi  # noqa: E402
from intel_gaudi3_software_b200.abi import make_tensor as T  # noqa: E402
from intel_gaudi3_software_b200.multi_gpu import ShardedCalculator, shard_range  # noqa: E402


def test_shard_range_partitions_exactly():
    for total in (0, 1, 7, 64, 8192, 200704):
        for world in (1, 2, 3, 8):
            spans = [shard_range(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


class OracleCalc:
    """Stand-in for Calculator with the same method names, computing with the CPU oracle."""

    def __init__(self):
        from oracle import Port
        self.port = Port()
        self.lib, self.ctx = None, None

    def do_batch_gemm(self, out, x, w, op, cast=None):
        assert self.port.bgemm(out, x, w, op, threads=1) == 0

    def do_convolution(self, out, x, w, y, params, op, rm=0, cast=None):
        assert self.port.conv(out, x, w, y, params, op, rm, threads=1) == 0


def worker(rank, world, port_no, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port_no))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import util
    rng = np.random.default_rng(0)  # every rank holds the same full tensors; shards are views
    sc = ShardedCalculator(OracleCalc(), dist, rank, world)
    # --- GEMM sharded over rows: no collective, rank r fills rows [b, e)
    M, N, K = 11, 6, 16
    xb, wb = util.gen_bf16(rng, M * K), util.gen_bf16(rng, K * N)
    out = np.zeros(M * N, np.float32)
    b, e = sc.batch_gemm_rows(T(out, abi.FP32, [N, M]), T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, [N, K]), abi.OP_AB)
    full = np.zeros(M * N, np.float32)
    OracleCalc().do_batch_gemm(T(full, abi.FP32, [N, M]), T(xb, abi.BF16, [K, M]), T(wb, abi.BF16, [N, K]), abi.OP_AB)
    ok_rows = (out.reshape(M, N)[b:e] == full.reshape(M, N)[b:e]).all() and (out.reshape(M, N)[:b] == 0).all() and (out.reshape(M, N)[e:] == 0).all()
    # --- conv fwd sharded over images
    xs, ws, ys = [4, 5, 4, 3], [3, 4, 3, 3], [3, 5, 4, 3]
    cx, cw, cy = util.gen_bf16(rng, int(np.prod(xs)), "normal"), util.gen_bf16(rng, int(np.prod(ws)), "normal", 0.1), util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.1)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    yo = np.zeros(int(np.prod(ys)), np.float32)
    ib, ie = sc.conv_images(T(yo, abi.FP32, ys), T(cx, abi.BF16, xs), T(cw, abi.BF16, ws), T(cy, abi.BF16, ys), cp, abi.OP_FWD)
    yfull = np.zeros(int(np.prod(ys)), np.float32)
    OracleCalc().do_convolution(T(yfull, abi.FP32, ys), T(cx, abi.BF16, xs), T(cw, abi.BF16, ws), T(cy, abi.BF16, ys), cp, abi.OP_FWD)
    per = int(np.prod(ys[:3]))
    ok_conv = (yo[ib * per: ie * per] == yfull[ib * per: ie * per]).all()
    # --- dedw: partials per rank, summed by a real all-reduce
    partial = torch.zeros(int(np.prod(ws)), dtype=torch.float32)
    pt = T(partial.numpy(), abi.FP32, ws)
    sc.conv_dedw(pt, T(cx, abi.BF16, xs), T(cw, abi.BF16, ws), T(cy, abi.BF16, ys), cp, lambda: dist.all_reduce(partial))
    wfull = np.zeros(int(np.prod(ws)), np.float32)
    OracleCalc().do_convolution(T(wfull, abi.FP32, ws), T(cx, abi.BF16, xs), T(cw, abi.BF16, ws), T(cy, abi.BF16, ys), cp, abi.OP_DEDW)
    # summing per-rank partials reorders the reduction: equal within the accumulator tolerance, not bitwise
    ok_dedw = np.abs(partial.numpy() - wfull).max() <= 2e-5 * np.abs(wfull).max()
    results[rank] = (bool(ok_rows), bool(ok_conv), bool(ok_dedw), (b, e), (ib, ie))
    dist.barrier()
    dist.destroy_process_group()


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.timeout(180)
def test_world_size_2_gloo():
    world = 2
    mgr = mp.Manager()
    results = mgr.dict()
    mp.spawn(worker, args=(world, free_port(), results), nprocs=world, join=True)
    assert len(results) == world
    for r in range(world):
        ok_rows, ok_conv, ok_dedw, rows, imgs = results[r]
        assert ok_rows and ok_conv and ok_dedw, (r, results[r])
    assert results[0][3] == (0, 6) and results[1][3] == (6, 11)
    assert results[0][4] == (0, 2) and results[1][4] == (2, 3)
