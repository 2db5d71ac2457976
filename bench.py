#!/usr/bin/env python
"""Benchmark of the MME compute path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the hot path over one batch of seeded synthetic input. The default workload is
the configuration the headline metric is quoted on: an fp8_143 (E4M3, exponent bias 7) GEMM with
M=N=K=8192, fp32 accumulation and a round-to-nearest-even bf16 output. With N > 1 ranks (launched by
torch.distributed.run, one process per GPU) every rank multiplies its own 8192-row shard of A by a
replica of B, so the job has M = 8192*N rows ("weak" scaling, no data-path collective); the dedw
workload is the one with a real exchange (an NCCL all-reduce of the fp32 partial weight gradients).

Rank 0 prints one JSON line. `value` is timed with operands resident in HBM; `e2e` is the same metric
through the C ABI with host buffers (pinned), host<->device copies inside the timed region.
`--impl reference` times the reference's own CPU calculator (oracle/_ref when built, else the C
restatement) on a bounded sample of the same workload, on the host cores.
"""
import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from intel_gaudi3_software_b200 import abi  # noqa: E402
from intel_gaudi3_software_b200.abi import make_tensor as T  # noqa: E402

L2_BYTES = 126 * 1024 * 1024

# name -> description of one step. FLOPs = 2*M*N*K; algorithmic bytes = operands read once +
# output written once in its final type.
WORKLOADS = {
    "fp8_gemm_8192": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                          out_dtype=abi.BF16, bound="tensor", peak_scale=2.0, dtype="fp8_143"),
    "fp8_gemm_8192_bias11": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=11,
                                 out_dtype=abi.BF16, bound="tensor", peak_scale=2.0, dtype="fp8_143"),
    # config 2 with the seeded stochastic-rounding cast (counter-based stream, fused into the epilogue)
    "fp8_gemm_8192_sr": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                             out_dtype=abi.BF16, bound="tensor", peak_scale=2.0, dtype="fp8_143", stochastic=True),
    # config 2 with fp8_143 output: round-to-nearest-even + clipping (hardware conversion), and stochastic rounding
    "fp8_gemm_8192_fp8out": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                                 out_dtype=abi.FP8_143, bound="tensor", peak_scale=2.0, dtype="fp8_143", clip=True),
    "fp8_gemm_8192_fp8out_sr": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                                    out_dtype=abi.FP8_143, bound="tensor", peak_scale=2.0, dtype="fp8_143", stochastic=True),
    "bf16_gemm_8192": dict(kind="gemm", M=8192, N=8192, K=8192, in_dtype=abi.BF16, w_dtype=abi.BF16, bias=0,
                           out_dtype=abi.BF16, bound="tensor", peak_scale=1.0, dtype="bf16"),
    "bf16_gemm_1024": dict(kind="gemm", M=1024, N=1024, K=1024, in_dtype=abi.BF16, w_dtype=abi.BF16, bias=0,
                           out_dtype=abi.FP32, bound="tensor", peak_scale=1.0, dtype="bf16"),
    "fp8_bgemm_attn": dict(kind="gemm", M=4096, N=4096, K=128, batch=64, op=abi.OP_ABT, in_dtype=abi.FP8_143,
                           w_dtype=abi.FP8_143, bias=7, out_dtype=abi.BF16, bound="hbm", peak_scale=2.0, dtype="fp8_143"),
    "fp8_mlp": dict(kind="gemm", M=16384, N=28672, K=8192, in_dtype=abi.FP8_152, w_dtype=abi.FP8_143, bias=7,
                    out_dtype=abi.BF16, bound="tensor", peak_scale=2.0, dtype="fp8_152xfp8_143"),
    # the optional bit-exact Gaudi3 accumulation (integer emulation on the CUDA cores; no tensor cores)
    "fp8_gemm_2048_exact": dict(kind="gemm", M=2048, N=2048, K=2048, in_dtype=abi.FP8_143, w_dtype=abi.FP8_143, bias=7,
                                out_dtype=abi.FP32, bound="tensor", peak_scale=2.0, dtype="fp8_143", exact=True),
    "conv_fwd": dict(kind="conv", op=abi.OP_FWD, out_dtype=abi.BF16, bound="tensor", peak_scale=1.0, dtype="bf16"),
    "conv_dedx": dict(kind="conv", op=abi.OP_DEDX, out_dtype=abi.BF16, bound="tensor", peak_scale=1.0, dtype="bf16"),
    "conv_dedw": dict(kind="conv", op=abi.OP_DEDW, out_dtype=abi.FP32, bound="tensor", peak_scale=1.0, dtype="bf16"),
    # same convolution, the cross-GPU sum fused into the split-K reduction (peer stores + rank-ordered gather)
    "conv_dedw_fused": dict(kind="conv", op=abi.OP_DEDW, out_dtype=abi.FP32, bound="tensor", peak_scale=1.0, dtype="bf16",
                            fused_exchange=True),
}
# HBM-bound helper kernels of the path (cast, comparator, memory-write reduction, tensor generator): one pass over n elements.
# value = algorithmic GB/s (bytes each kernel must read and write once); they run on tensors far larger than L2.
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

# DRAM bytes per launch of the dominant kernel from an ncu capture (profiles/*.md say which
# command produced each number); None where no capture exists yet.
NCU_TRAFFIC_BYTES = {
    "fp8_gemm_8192": 357.2e6,        # profiles/gemm_tcgen05_pair_fp8_gemm_8192.md
    "fp8_gemm_8192_bias11": 357.2e6,  # same kernel and byte streams; only the epilogue scale differs
    "bf16_gemm_8192": 1346.8e6,      # profiles/gemm_tcgen05_pair_other_workloads.md
    "conv_fwd": 165.8e6,
    "conv_dedx": 165.5e6,
    "conv_dedw": 210.2e6,
    "fp8_bgemm_attn": 2155.1e6,
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(hbm=d["hbm_gbs"], bf16=d["bf16_tflops"], bf16_sustained=d.get("bf16_tflops_sustained", d["bf16_tflops"]),
                    source="measured")
    return dict(hbm=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.proc = None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        clocks, mx, reasons = [], None, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        # the busiest samples are the ones under load
        clocks.sort()
        load = clocks[len(clocks) // 2:] if clocks else []
        return {"sm_mhz": statistics.median(load) if load else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(clocks)}


def conv_shapes():
    c = CONV
    xs = [c["C"], c["W"], c["H"], c["B"]]
    ws = [c["K"], c["C"], c["S"], c["R"]]
    ys = [c["K"], c["W"], c["H"], c["B"]]
    return xs, ws, ys


def workload_counts(wl):
    """(flops, algorithmic bytes, units description) of one step."""
    if wl["kind"] == "gemm":
        b = wl.get("batch", 1)
        M, N, K = wl["M"], wl["N"], wl["K"]
        flops = 2.0 * M * N * K * b
        byts = b * (M * K * abi.ELEM_SIZE[wl["in_dtype"]] + K * N * abi.ELEM_SIZE[wl["w_dtype"]] +
                    M * N * abi.ELEM_SIZE[wl["out_dtype"]])
        return flops, float(byts)
    xs, ws, ys = conv_shapes()
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


def synth_inputs(wl, seed, rows=None):
    """Seeded synthetic operands with the configuration's shapes and value distributions.

    fp8 operands: N(0,1) scaled per tensor to amax = the format's largest finite value, RNE-cast.
    Generated directly as code bytes from a normal draw through a numpy quantiser that reproduces
    the RNE cast for in-range values (checked against the oracle in tests/test_bench_inputs.py).
    """
    import util
    rng = np.random.default_rng(seed)
    if wl["kind"] == "gemm":
        b = wl.get("batch", 1)
        M = rows if rows is not None else wl["M"]
        N, K = wl["N"], wl["K"]

        def make(n, dtype, bias):
            if dtype == abi.BF16:
                return util.f32_to_bf16_rne(rng.uniform(-1, 1, n).astype(np.float32))
            return quantise_fp8(rng.standard_normal(n, dtype=np.float32), dtype, bias)
        x = make(M * K * b, wl["in_dtype"], wl["bias"] if wl["in_dtype"] == abi.FP8_143 else 15)
        w = make(K * N * b, wl["w_dtype"], 7 if wl["w_dtype"] == abi.FP8_143 and wl["in_dtype"] != abi.FP8_143 else wl["bias"])
        return x, w
    xs, ws, ys = conv_shapes()
    x = util.f32_to_bf16_rne(rng.standard_normal(int(np.prod(xs)), dtype=np.float32))
    w = util.f32_to_bf16_rne((rng.standard_normal(int(np.prod(ws)), dtype=np.float32) * np.float32(np.sqrt(2.0 / (ws[1] * ws[2] * ws[3])))))
    y = util.f32_to_bf16_rne((rng.standard_normal(int(np.prod(ys)), dtype=np.float32) * np.float32(0.01)))
    return x, w, y


def quantise_fp8(v, dtype, bias):
    """RNE cast of N(0,1) draws, scaled to amax = max finite, to fp8 code bytes (numpy, vectorised).

    1-4-3 uses the 'minimal Inf/NaN' convention (max 448 * 2^(7-bias)); 1-5-2 the full one (max 57344 * 2^(15-bias)).
    """
    man = 3 if dtype == abi.FP8_143 else 2
    hw_bias = 7 if dtype == abi.FP8_143 else 15
    maxv = (448.0 if dtype == abi.FP8_143 else 57344.0)
    a = v * np.float32(maxv / np.abs(v).max())          # in hardware-bias units; the tensor's bias only rescales
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


def dist_setup(n_gpus):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        return rank, world, local, dist
    return rank, world, local, None


def barrier_and_max(dist, value, local):
    if dist is None:
        return value
    import torch
    t = torch.tensor([value], dtype=torch.float64, device=torch.device("cuda", local))
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_stream(args):
    """One of the HBM-bound helper kernels on device-resident tensors (single GPU)."""
    import intel_gaudi3_software_b200 as pkg
    wl = WORKLOADS[args.workload]
    calc = pkg.Calculator(device=0)
    n = wl["n"]
    dev = abi.MEM_DEVICE
    bufs = []

    def alloc(nbytes):
        b = calc.alloc(nbytes)
        bufs.append(b)
        return b
    if args.workload == "cast_f32_to_bf16":
        src, dst = alloc(n * 4), alloc(n * 2)
        calc.generate(T(src.ptr, abi.FP32, [n], mem_space=dev), abi.GEN_NORMAL, -100.0, 100.0, 0.0, 1.0, seed=1)
        cp = abi.make_cast_params(abi.RM_NE)
        step = lambda: calc.do_activation(T(dst.ptr, abi.BF16, [n], mem_space=dev), T(src.ptr, abi.FP32, [n], mem_space=dev), cp)  # noqa: E731
    elif args.workload in ("cast_f32_to_fp8", "cast_f32_to_bf16_sr"):
        fp8 = args.workload == "cast_f32_to_fp8"
        src, dst = alloc(n * 4), alloc(n * (1 if fp8 else 2))
        calc.generate(T(src.ptr, abi.FP32, [n], mem_space=dev), abi.GEN_NORMAL, -100.0, 100.0, 0.0, 1.0, seed=1)
        cp = abi.make_cast_params(abi.RM_NE, clip_fp=True) if fp8 else abi.make_cast_params(abi.RM_SR, rng_kind=abi.RNG_PHILOX, rng_seed=9)
        to = T(dst.ptr, abi.FP8_143, [n], fp_bias=7, inf_nan_mode=abi.INFNAN_MINIMAL, mem_space=dev) if fp8 else T(dst.ptr, abi.BF16, [n], mem_space=dev)
        step = lambda: calc.do_activation(to, T(src.ptr, abi.FP32, [n], mem_space=dev), cp)  # noqa: E731
    elif args.workload == "compare_bf16":
        a, b = alloc(n * 2), alloc(n * 2)
        for buf, seed in ((a, 1), (b, 1)):
            calc.generate(T(buf.ptr, abi.BF16, [n], mem_space=dev), abi.GEN_UNIFORM, -4.0, 4.0, seed=seed)
        step = lambda: calc.compare(T(a.ptr, abi.BF16, [n], mem_space=dev), T(b.ptr, abi.BF16, [n], mem_space=dev), 4096)  # noqa: E731
    elif args.workload == "memory_write_add_f32":
        mem, src = alloc(n * 4), alloc(n * 4)
        calc.generate(T(mem.ptr, abi.FP32, [n], mem_space=dev), abi.GEN_FILL, 0.0, 0.0)
        calc.generate(T(src.ptr, abi.FP32, [n], mem_space=dev), abi.GEN_UNIFORM, -1.0, 1.0, seed=2)
        step = lambda: calc.do_memory_write(T(mem.ptr, abi.FP32, [n], mem_space=dev), T(src.ptr, abi.FP32, [n], mem_space=dev), abi.RED_ADD, 0)  # noqa: E731
    else:
        out = alloc(n * 2)
        step = lambda: calc.generate(T(out.ptr, abi.BF16, [n], mem_space=dev), abi.GEN_UNIFORM, -1.0, 1.0, seed=3)  # noqa: E731
    steps = min(args.steps, 50)
    for _ in range(max(args.warmup, 3)):
        step()
    calc.sync()
    launches0 = calc.launch_count()
    sampler = ClockSampler(0)
    calc.timer_start()
    for _ in range(steps):
        step()
    ms = calc.timer_stop() / steps
    clocks = sampler.stop()
    launches = calc.launch_count() - launches0
    peaks = measured_peaks()
    alg = float(n) * wl["bytes_per_elem"]
    gbs = alg / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "HBM GB/s (algorithmic bytes)", "value": gbs, "unit": "GB/s", "n_gpus": 1, "steps": steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, "elements": n, "l2": "tensors of %d MiB exceed the 126 MB L2" % (alg / 2**20)},
        "gpu_launches": launches, "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm"], "unit": "GB/s", "frac": gbs / peaks["hbm"], "traffic": None,
                     "peak_note": "%s copy bandwidth" % peaks["source"], "algorithmic_bytes_per_launch": alg},
    }))
    for b in bufs:
        b.free()
    calc.close()


def run_ours(args):
    import intel_gaudi3_software_b200 as pkg
    wl = WORKLOADS[args.workload]
    if wl["kind"] == "stream":
        return run_stream(args)
    rank, world, local, dist = dist_setup(args.gpus)
    calc = pkg.Calculator(device=local)
    if wl.get("exact"):
        calc.set_accumulation(abi.ACC_CHIP_EXACT)
    lib, ctx = calc.lib, calc.ctx
    flops, alg_bytes = workload_counts(wl)
    cast = abi.make_cast_params(abi.RM_NE) if wl["out_dtype"] != abi.FP32 else None
    if wl.get("stochastic"):
        cast = abi.make_cast_params(abi.RM_SR, clip_fp=True, rng_kind=abi.RNG_PHILOX, rng_seed=2024)
    elif wl.get("clip"):
        cast = abi.make_cast_params(abi.RM_NE, clip_fp=True)

    # ---- operands, resident in HBM (each rank: its own shard, seeded by rank)
    host = synth_inputs(wl, seed=1000 + rank)
    dev = [calc.to_device(h) for h in host]
    if wl["kind"] == "gemm":
        b = wl.get("batch", 1)
        M, N, K = wl["M"], wl["N"], wl["K"]
        op = wl.get("op", abi.OP_AB)
        bdims = [b] if b > 1 else []
        xs = [K, M] + bdims
        ws = ([K, N] if op == abi.OP_ABT else [N, K]) + bdims
        os_ = [N, M] + bdims
        x_bias = wl["bias"] if wl["in_dtype"] == abi.FP8_143 else 15
        w_bias = 7 if wl["in_dtype"] != abi.FP8_143 else wl["bias"]
        mode = lambda dt: abi.INFNAN_MINIMAL if dt == abi.FP8_143 else abi.INFNAN_FULL  # noqa: E731
        out_bytes = int(np.prod(os_)) * abi.ELEM_SIZE[wl["out_dtype"]]
        dout = calc.alloc(out_bytes)

        def tensors(px, pw, po, space):
            return (T(po, wl["out_dtype"], os_, fp_bias=7 if wl["out_dtype"] == abi.FP8_143 else 15, inf_nan_mode=mode(wl["out_dtype"]), mem_space=space),
                    T(px, wl["in_dtype"], xs, fp_bias=x_bias, inf_nan_mode=mode(wl["in_dtype"]), mem_space=space),
                    T(pw, wl["w_dtype"], ws, fp_bias=w_bias, inf_nan_mode=mode(wl["w_dtype"]), mem_space=space))
        to, tx, tw = tensors(dev[0].ptr, dev[1].ptr, dout.ptr, abi.MEM_DEVICE)

        def step():
            calc.do_batch_gemm(to, tx, tw, op, cast)
        in_bytes = host[0].nbytes + host[1].nbytes
    else:
        xs, ws, ys = conv_shapes()
        cp = abi.make_conv_params(2, (CONV["pad"], CONV["pad"]), (1, 1), (1, 1))
        oshape = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[wl["op"]]
        out_bytes = int(np.prod(oshape)) * abi.ELEM_SIZE[wl["out_dtype"]]
        dout = calc.alloc(out_bytes)

        def tensors(px, pw, py, po, space):
            return (T(po, wl["out_dtype"], oshape, mem_space=space), T(px, abi.BF16, xs, mem_space=space),
                    T(pw, abi.BF16, ws, mem_space=space), T(py, abi.BF16, ys, mem_space=space))
        to, tx, tw, ty = tensors(dev[0].ptr, dev[1].ptr, dev[2].ptr, dout.ptr, abi.MEM_DEVICE)
        overlap = None
        exchange = None
        if wl.get("fused_exchange"):
            from intel_gaudi3_software_b200.multi_gpu import PeerExchange
            exchange = PeerExchange(calc, int(np.prod(oshape)), dist, rank, world, deferred_output=True)
        elif wl["op"] == abi.OP_DEDW and dist is not None:
            # dW partials are all-reduced over NCCL on a second stream, double-buffered, so that the
            # exchange of step i overlaps the convolution of step i+1 (as it would overlap the next
            # layer's work in a training step)
            import torch
            dev_t = torch.device("cuda", local)
            bufs = [torch.empty(int(np.prod(oshape)), dtype=torch.float32, device=dev_t) for _ in range(2)]
            tos = [T(b.data_ptr(), abi.FP32, oshape, mem_space=abi.MEM_DEVICE) for b in bufs]
            comm = torch.cuda.Stream(device=dev_t)
            main = torch.cuda.current_stream(dev_t)
            calc.set_stream(main.cuda_stream)
            overlap = dict(i=0, done=[None, None])

        def step():
            if exchange is not None:
                exchange.dedw_allreduce(to, tx, tw, ty, cp)
                return
            if overlap is None:
                calc.do_convolution(to, tx, tw, ty, cp, wl["op"], abi.RM_NE, cast)
                return
            k = overlap["i"] & 1
            overlap["i"] += 1
            if overlap["done"][k] is not None:
                main.wait_event(overlap["done"][k])      # buffer k is free once its all-reduce finished
            calc.do_convolution(tos[k], tx, tw, ty, cp, wl["op"], abi.RM_NE, cast)
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                dist.all_reduce(bufs[k])
                ev = torch.cuda.Event()
                ev.record(comm)
            overlap["done"][k] = ev
        used = {abi.OP_FWD: (0, 1), abi.OP_DEDX: (2, 1), abi.OP_DEDW: (0, 2)}[wl["op"]]
        in_bytes = sum(host[i].nbytes for i in used)

    # ---- device-resident timing
    for _ in range(max(args.warmup, 3)):
        step()
    calc.sync()
    launches0 = calc.launch_count()
    barrier_and_max(dist, 0.0, local)
    sampler = ClockSampler(local) if rank == 0 else None
    calc.sync()
    calc.timer_start()
    for _ in range(args.steps):
        step()
    if wl["kind"] == "conv" and overlap is not None:
        for ev in overlap["done"]:
            if ev is not None:
                main.wait_event(ev)                      # the timed region ends when the last exchange has
    ms = calc.timer_stop()
    calc.sync()
    clocks = sampler.stop() if sampler else None
    launches = calc.launch_count() - launches0
    ms = barrier_and_max(dist, ms, local)
    ms_per_step = ms / args.steps
    value = world * flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the C ABI with pinned host buffers
    def pinned(nbytes):
        p = C.c_void_p()
        assert lib.mmeb200_host_alloc(C.byref(p), nbytes) == 0
        return p.value
    e2e_steps = max(3, min(args.steps, 10))
    hp = []
    for h in host:
        p = pinned(h.nbytes)
        C.memmove(p, h.ctypes.data, h.nbytes)
        hp.append(p)
    hout = pinned(out_bytes)
    if wl["kind"] == "gemm":
        eo, ex, ew = tensors(hp[0], hp[1], hout, abi.MEM_HOST)

        def e2e_step():
            calc.do_batch_gemm(eo, ex, ew, op, cast)
    else:
        eo, ex, ew, ey = tensors(hp[0], hp[1], hp[2], hout, abi.MEM_HOST)

        def e2e_step():
            calc.do_convolution(eo, ex, ew, ey, cp, wl["op"], abi.RM_NE, cast)
    if wl["kind"] == "conv":
        calc.set_stream(None)
    for _ in range(2):   # the first host-tensor calls size the library's staging arena
        e2e_step()
    calc.sync()
    barrier_and_max(dist, 0.0, local)
    calc.timer_start()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_ms = calc.timer_stop() / e2e_steps
    e2e_ms = barrier_and_max(dist, e2e_ms, local)
    e2e_value = world * flops / (e2e_ms * 1e-3) / 1e12
    result_checksum = int(np.frombuffer((C.c_uint8 * min(out_bytes, 4096)).from_address(hout), dtype=np.uint8).sum())

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peaks = measured_peaks()
    total_s = ms * 1e-3
    sustained = total_s > 1.0
    if wl["bound"] == "tensor":
        base = peaks["bf16_sustained"] if sustained else peaks["bf16"]
        peak = base * wl["peak_scale"]
        achieved = flops / (ms_per_step * 1e-3) / 1e12
        unit = "TFLOP/s"
        note = "%s bf16 cuBLAS %s figure%s" % (peaks["source"], "sustained" if sustained else "burst",
                                                " x2 for fp8 (no fp8 figure in MEASURED_PEAKS.json)" if wl["peak_scale"] == 2.0 else "")
    else:
        peak = peaks["hbm"]
        achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
        unit = "GB/s"
        note = "%s HBM copy bandwidth" % peaks["source"]
    line = {
        "metric": "GEMM/conv TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, "per_gpu": {k: v for k, v in wl.items() if k in ("M", "N", "K", "batch")} or CONV,
                   "accumulate": "Gaudi3 tree, bit-exact (integer emulation, no tensor cores: the tensor peak is shown for scale only)" if wl.get("exact") else "fp32",
                   "output": {abi.BF16: "bf16", abi.FP8_143: "fp8_143", abi.FP32: "fp32"}[wl["out_dtype"]] +
                             ("" if wl["out_dtype"] == abi.FP32 else " stochastic rounding (Philox)" if wl.get("stochastic") else
                              " RNE + clip" if wl.get("clip") else " RNE"),
                   "l2": "operands + output (%d MiB) exceed the 126 MB L2; no flush between steps" % ((in_bytes + out_bytes) >> 20)
                   if in_bytes + out_bytes > L2_BYTES else "working set fits L2 (latency-bound correctness config)",
                   "sharding": "rows of A / images per rank, replica of B / weights" if wl.get("op") != abi.OP_DEDW else
                   ("reduction dim sharded; fp32 partials exchanged by the reduction kernel itself over peer memory"
                    if wl.get("fused_exchange") else "reduction dim sharded; fp32 partials all-reduced over NCCL (overlapped)")},
        "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": in_bytes, "d2h_bytes_per_step": out_bytes,
                "ms_per_step": e2e_ms, "result_checksum": result_checksum},
        "gpu_launches": launches,
        "clocks": clocks,
        "roofline": {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
                     "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "peak_note": note,
                     "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": alg_bytes},
    }
    if world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(wl, args.workload, budget_s=12.0)
    print(json.dumps(line))


_CPU_W_CACHE = {}


def cpu_sample(wl, rows_hint=None):
    """Bounded sample of the workload for the CPU calculator: a block of A's rows against all of B
    (whole common dimension), or a few output rows of the convolution's GEMM."""
    from oracle import Port, Ref, have_ref
    lib = Ref() if have_ref() else Port()
    threads = lib.hardware_threads()
    return lib, threads


def cpu_run(lib, wl, rows, threads, seed=1000):
    """One bounded CPU sample; returns (seconds, flops)."""
    if wl["kind"] == "gemm":
        import util
        N, K = wl["N"], wl["K"]
        key = (wl["w_dtype"], N, K, seed)
        if key not in _CPU_W_CACHE:   # B is the same for every sample of a run: draw it once
            r = np.random.default_rng(seed + 1)
            _CPU_W_CACHE[key] = (util.f32_to_bf16_rne(r.uniform(-1, 1, K * N).astype(np.float32)) if wl["w_dtype"] == abi.BF16
                                 else quantise_fp8(r.standard_normal(K * N, dtype=np.float32), wl["w_dtype"], 7))
        w = _CPU_W_CACHE[key]
        r = np.random.default_rng(seed)
        x = (util.f32_to_bf16_rne(r.uniform(-1, 1, rows * K).astype(np.float32)) if wl["in_dtype"] == abi.BF16
             else quantise_fp8(r.standard_normal(rows * K, dtype=np.float32), wl["in_dtype"], 7))
        x_bias = wl["bias"] if wl["in_dtype"] == abi.FP8_143 else 15
        w_bias = 7 if wl["in_dtype"] != abi.FP8_143 else wl["bias"]
        mode = lambda dt: abi.INFNAN_MINIMAL if dt == abi.FP8_143 else abi.INFNAN_FULL  # noqa: E731
        acc = np.zeros(rows * N, np.float32)
        out = np.zeros(rows * N, abi.NP_DTYPE[wl["out_dtype"]])
        # the CPU sample uses the 'ab' orientation; the arithmetic per output is the same
        tx = T(x, wl["in_dtype"], [K, rows], fp_bias=x_bias, inf_nan_mode=mode(wl["in_dtype"]))
        tw = T(w, wl["w_dtype"], [N, K], fp_bias=w_bias, inf_nan_mode=mode(wl["w_dtype"]))
        t0 = time.perf_counter()
        rc = lib.bgemm(T(acc, abi.FP32, [N, rows]), tx, tw, abi.OP_AB, threads=threads)
        assert rc == 0
        if wl["out_dtype"] != abi.FP32:
            lib.fp32_to_bf16(acc)
        dt = time.perf_counter() - t0
        return dt, 2.0 * rows * N * K
    # convolution: one image with `rows` output rows of the 56x56 grid is not expressible; use whole small images
    c = dict(CONV, B=1, H=rows, W=CONV["W"])
    xs, ws, ys = [c["C"], c["W"], c["H"], 1], [c["K"], c["C"], c["S"], c["R"]], [c["K"], c["W"], c["H"], 1]
    import util
    rng = np.random.default_rng(seed)
    x = util.f32_to_bf16_rne(rng.standard_normal(int(np.prod(xs)), dtype=np.float32))
    w = util.f32_to_bf16_rne(rng.standard_normal(int(np.prod(ws)), dtype=np.float32) * np.float32(0.0295))
    y = util.f32_to_bf16_rne(rng.standard_normal(int(np.prod(ys)), dtype=np.float32) * np.float32(0.01))
    oshape = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[wl["op"]]
    acc = np.zeros(int(np.prod(oshape)), np.float32)
    cp = abi.make_conv_params(2, (1, 1), (1, 1), (1, 1))
    t0 = time.perf_counter()
    rc = lib.conv(T(acc, abi.FP32, oshape), T(x, abi.BF16, xs), T(w, abi.BF16, ws), T(y, abi.BF16, ys), cp, wl["op"],
                  threads=threads)
    assert rc == 0
    dt = time.perf_counter() - t0
    return dt, 2.0 * ys[1] * ys[2] * ws[0] * ws[1] * ws[2] * ws[3]


def pick_rows(lib, wl, threads, budget_s):
    """Calibrate on a tiny sample, then size the bounded sample to about budget_s of CPU work."""
    probe = max(2, threads) if wl["kind"] == "gemm" else 2   # one row per thread: the probe sees the parallel rate
    dt, fl = cpu_run(lib, wl, probe, threads)
    per_row = dt / probe
    rows = int(max(probe, min(budget_s / max(per_row, 1e-6), 4096 if wl["kind"] == "gemm" else CONV["H"])))
    if wl["kind"] == "gemm":
        rows = max(threads, (rows // threads) * threads) if rows >= threads else rows
    return rows


def cpu_baseline(wl, name, budget_s):
    lib, threads = cpu_sample(wl)
    rows = pick_rows(lib, wl, threads, budget_s)
    dt, fl = cpu_run(lib, wl, rows, threads)
    sample = ("%d rows of A x all of B (K whole)" % rows) if wl["kind"] == "gemm" else ("one image of %d x %d pixels" % (rows, CONV["W"]))
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": lib.kind, "sample": sample,
            "seconds": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    lib, threads = cpu_sample(wl)
    # size one step so that warmup + steps end within a few minutes
    total_budget = 150.0
    per_step = total_budget / max(1, args.steps + args.warmup)
    rows = pick_rows(lib, wl, threads, min(per_step, 20.0))
    for _ in range(args.warmup):
        cpu_run(lib, wl, rows, threads)
    t, fl = 0.0, 0.0
    for _ in range(args.steps):
        dt, f = cpu_run(lib, wl, rows, threads)
        t += dt
        fl += f
    value = fl / t / 1e12
    sample = ("%d rows of A x all of B (K whole)" % rows) if wl["kind"] == "gemm" else ("one image of %d x %d pixels" % (rows, CONV["W"]))
    line = {
        "impl": "reference", "metric": "GEMM/conv TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": {"workload": args.workload, "per_gpu": {k: v for k, v in wl.items() if k in ("M", "N", "K", "batch")} or CONV,
                   "accumulate": "fp32", "note": "reference CPU calculator on the host cores; each step is a bounded sample: " + sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": lib.kind, "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="fp8_gemm_8192", choices=sorted(WORKLOADS))
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="leave the CPU baseline leg out (sweeps)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
