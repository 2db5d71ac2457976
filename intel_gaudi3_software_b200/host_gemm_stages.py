"""Per-stage host timers of the multi-GPU host-tensor GEMM (ShardedCalculator.host_gemm_shared_b) on the fp8 8192^3
configuration: this rank's 1/N of B over PCIe, the NCCL all-gather of B, and the library's row-block pipeline around the
resident B (pipelined on the caller's stream, not pipelined, pipelined on the library's own stream). One process per GPU:

    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 --master-port P \\
        -m intel_gaudi3_software_b200.host_gemm_stages
"""
import ctypes as C
import os
import time

import torch
import torch.distributed as dist

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
from intel_gaudi3_software_b200.multi_gpu import ShardedCalculator


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    calc = pkg.Calculator(device=local)
    lib = calc.lib
    M, N, K = 8192 // world, 8192, 8192
    def pinned(n):
        p = C.c_void_p(); assert lib.mmeb200_host_alloc(C.byref(p), n) == 0; return p.value
    ha, hb, ho = pinned(M * K), pinned(K * N), pinned(M * N * 2)
    C.memset(ha, 0x38, M * K); C.memset(hb, 0x38, K * N)
    kw = dict(fp_bias=7, inf_nan_mode=2)
    eo, ex, ew = T(ho, abi.BF16, [N, M]), T(ha, abi.FP8_143, [K, M], **kw), T(hb, abi.FP8_143, [N, K], **kw)
    cast = abi.make_cast_params(abi.RM_NE)
    sc = ShardedCalculator(calc, dist, rank, world, device=local)
    def sync():
        torch.cuda.synchronize(); calc.sync()
    for _ in range(3): sc.host_gemm_shared_b(eo, ex, ew, abi.OP_AB, cast)
    sync(); dist.barrier()
    # whole
    t0 = time.perf_counter()
    for _ in range(10): sc.host_gemm_shared_b(eo, ex, ew, abi.OP_AB, cast)
    sync(); whole = (time.perf_counter() - t0) / 10 * 1e3
    # stages
    nbytes = K * N; piece = nbytes // world
    buf = sc._shared_b
    stream = torch.cuda.current_stream()
    calc.set_stream(stream.cuda_stream)
    def timed(fn, reps=10):
        sync(); dist.barrier(); t0 = time.perf_counter()
        for _ in range(reps): fn()
        sync(); return (time.perf_counter() - t0) / reps * 1e3
    t_h2d = timed(lambda: calc._check(lib.mmeb200_memcpy_h2d(calc.ctx, buf.data_ptr() + rank * piece, hb + rank * piece, piece)))
    t_gather = timed(lambda: dist.all_gather_into_tensor(buf, buf[rank * piece:(rank + 1) * piece]))
    wd = abi.Tensor(); C.memmove(C.byref(wd), C.byref(ew), C.sizeof(abi.Tensor)); wd.data, wd.mem_space = buf.data_ptr(), abi.MEM_DEVICE
    t_gemm = timed(lambda: calc.do_batch_gemm(eo, ex, wd, abi.OP_AB, cast))
    calc.set_option("host_pipeline", 0)
    t_gemm_nopipe = timed(lambda: calc.do_batch_gemm(eo, ex, wd, abi.OP_AB, cast))
    calc.set_option("host_pipeline", -1)
    calc.set_stream(None)
    t_gemm_own_stream = timed(lambda: calc.do_batch_gemm(eo, ex, wd, abi.OP_AB, cast))
    print("rank %d/%d: whole %.3f ms | B slice h2d %.3f | all_gather %.3f | gemm (host A, out; resident B) %.3f | same, not pipelined %.3f | pipelined on the library's own stream %.3f" % (rank, world, whole, t_h2d, t_gather, t_gemm, t_gemm_nopipe, t_gemm_own_stream), flush=True)
    dist.barrier(); calc.close(); dist.destroy_process_group()


if __name__ == "__main__":
    main()
