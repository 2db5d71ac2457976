"""One rank of the multi-GPU peer-exchange test (launched by torch.distributed.run, one process per GPU)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))
import intel_gaudi3_software_b200 as pkg  # noqa: E402
from intel_gaudi3_software_b200 import abi  # noqa: E402
from intel_gaudi3_software_b200.abi import make_tensor as T  # noqa: E402
from intel_gaudi3_software_b200.multi_gpu import PeerExchange, shard_range  # noqa: E402
import util  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    calc = pkg.Calculator(device=local)
    B = 2 * world
    xs, ws, ys = [64, 32, 32, B], [64, 64, 3, 3], [64, 32, 32, B]
    rng = np.random.default_rng(5)   # every rank draws the same full tensors
    xb = util.gen_bf16(rng, int(np.prod(xs)), "normal")
    yb = util.gen_bf16(rng, int(np.prod(ys)), "normal", 0.01)
    wb = np.zeros(int(np.prod(ws)), np.uint16)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    n = int(np.prod(ws))
    # the whole batch on one GPU: what the sum over ranks must equal (up to the order of summation)
    full, sabs = np.zeros(n, np.float32), np.zeros(n, np.float32)
    calc.do_convolution(T(full, abi.FP32, ws), T(xb, abi.BF16, xs), T(wb, abi.BF16, ws), T(yb, abi.BF16, ys), cp, abi.OP_DEDW)
    # sum|a_k b_k| per element: the same dedw on the operands' absolute values (the scale of the accumulator tolerance)
    calc.do_convolution(T(sabs, abi.FP32, ws), T(util.clear_signs(xb, abi.BF16), abi.BF16, xs), T(wb, abi.BF16, ws),
                        T(util.clear_signs(yb, abi.BF16), abi.BF16, ys), cp, abi.OP_DEDW)
    tol = util.ACC_TOL * sabs.astype(np.float64)
    b0, b1 = shard_range(B, world, rank)
    per_x, per_y = int(np.prod(xs[:3])), int(np.prod(ys[:3]))
    xs_r, ys_r = xs[:3] + [b1 - b0], ys[:3] + [b1 - b0]
    xr, yr = xb[b0 * per_x: b1 * per_x], yb[b0 * per_y: b1 * per_y]
    ex = PeerExchange(calc, n, dist, rank, world)
    ok = True
    for it in range(6):
        out = np.zeros(n, np.float32)
        ex.dedw_allreduce(T(out, abi.FP32, ws), T(xr, abi.BF16, xs_r), T(wb, abi.BF16, ws), T(yr, abi.BF16, ys_r), cp)
        ok &= bool((np.abs(out.astype(np.float64) - full) <= tol).all())
        # all ranks must hold bit-identical sums
        t = torch.from_numpy(out.view(np.int32).copy()).cuda()
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ok &= bool((lo == hi).all().item())
    dist.barrier()
    ex.close()
    # device-resident tensors with the deferred output: the final add of step i overlaps the convolution of step i+1
    ex2 = PeerExchange(calc, n, dist, rank, world, deferred_output=True)
    dx, dw, dy, dout = calc.to_device(xr), calc.to_device(wb), calc.to_device(yr), calc.alloc(n * 4)
    dev = abi.MEM_DEVICE
    for it in range(7):
        ex2.dedw_allreduce(T(dout.ptr, abi.FP32, ws, mem_space=dev), T(dx.ptr, abi.BF16, xs_r, mem_space=dev),
                           T(dw.ptr, abi.BF16, ws, mem_space=dev), T(dy.ptr, abi.BF16, ys_r, mem_space=dev), cp)
    calc.sync(10_000_000_000)
    out = dout.download(np.float32)
    ok &= bool((np.abs(out.astype(np.float64) - full) <= tol).all())
    t = torch.from_numpy(out.view(np.int32).copy()).cuda()
    lo, hi = t.clone(), t.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    ok &= bool((lo == hi).all().item())
    dist.barrier()
    ex2.close()
    # the bit-exact accumulation mode: exact partials per rank, same exchange, bit-identical sums on all ranks
    exact = pkg.Calculator(device=local, accumulation=abi.ACC_CHIP_EXACT)
    ex3 = PeerExchange(exact, n, dist, rank, world)
    for it in range(2):
        out = np.zeros(n, np.float32)
        ex3.dedw_allreduce(T(out, abi.FP32, ws), T(xr, abi.BF16, xs_r), T(wb, abi.BF16, ws), T(yr, abi.BF16, ys_r), cp)
        ok &= bool((np.abs(out.astype(np.float64) - full) <= tol).all())
        t = torch.from_numpy(out.view(np.int32).copy()).cuda()
        lo, hi = t.clone(), t.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        ok &= bool((lo == hi).all().item())
    dist.barrier()
    ex3.close()
    exact.close()
    calc.close()
    flag = torch.tensor([1 if ok else 0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    if rank == 0:
        print("PEER EXCHANGE OK" if flag.item() == 1 else "PEER EXCHANGE FAILED")
    dist.destroy_process_group()
    sys.exit(0 if flag.item() == 1 else 1)


if __name__ == "__main__":
    main()
