#!/usr/bin/env python
"""Benchmark of the MME compute path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]
                    [--scaling strong|weak] [--configs default|none]

A step is one pass of the hot path over one batch of seeded synthetic input. The default workload is the
configuration the headline metric is quoted on: an fp8_143 (E4M3, exponent bias 7) GEMM with M=N=K=8192, fp32
accumulation and a round-to-nearest-even bf16 output.

With N > 1 ranks (launched by torch.distributed.run, one process per GPU) the FIXED configuration is split over the
ranks ("strong" scaling, the default): GEMM rows of A / convolution images are sharded, B / the weights are replicated,
no collective is on the data path; dedw shards its reduction (the images) and sums the fp32 partial weight gradients
over NVLink inside the timed region (NCCL all-reduce, or the library's fused peer exchange). `--scaling weak` gives
every rank the whole per-GPU workload instead.

Rank 0 prints one JSON line:
  value      whole-job TFLOP/s with operands resident in HBM (CUDA events on the launching stream, max over ranks);
  sustained  the same launch back to back for at least two seconds, with the clocks sampled inside that window;
  e2e        the same metric through the public API with pinned HOST buffers, host<->device copies inside the timed
             region (N > 1: the multi-GPU driver uploads 1/N of B per rank and spreads it over NVLink);
  configs    every benchmark configuration timed the same way (device-resident), each with its roofline fraction;
  roofline   against the measured peaks (bf16: MEASURED_PEAKS.json; fp8: a cuBLASLt e4m3 GEMM timed in this run).
`--impl reference` times the reference's own CPU calculator (oracle/_ref when built, else the C restatement) on a
bounded sample of the same workload, on the host cores.
"""
import argparse
import ctypes as C
import datetime
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from intel_gaudi3_software_b200 import abi  # noqa: E402
from intel_gaudi3_software_b200.abi import make_tensor as T  # noqa: E402
from intel_gaudi3_software_b200 import workloads as W  # noqa: E402
from intel_gaudi3_software_b200.workloads import WORKLOADS, CONV, L2_BYTES  # noqa: E402

# configurations timed in the default run, beside the headline workload
DEFAULT_CONFIGS = ["bf16_gemm_1024", "fp8_gemm_8192", "fp8_gemm_8192_bias11", "fp8_gemm_8192_sr", "conv_fwd", "conv_dedx", "conv_dedw",
                   "fp8_bgemm_attn", "fp8_mlp", "bf16_gemm_8192", "fp32_gemm_4096", "tf32_gemm_4096"]
MULTI_GPU_CONFIGS = ["fp8_gemm_8192", "bf16_gemm_8192", "conv_fwd", "conv_dedx", "conv_dedw", "conv_dedw_fused"]

# DRAM bytes per launch of the dominant kernel from an ncu capture (profiles/*.md say which command produced each
# number); None where no capture exists.
NCU_TRAFFIC_BYTES = {
    "fp8_gemm_8192": 352.9e6,        # profiles/gemm_tcgen05_pair_fp8_gemm_8192.md
    "fp8_gemm_8192_bias11": 352.9e6,  # same kernel and byte streams; only the epilogue scale differs
    "fp8_gemm_8192_sr": 352.6e6,     # profiles/gemm_tcgen05_pair_epilogue_casts.md
    "fp8_gemm_8192_fp8out": 274.9e6,
    "fp8_gemm_8192_fp8out_sr": 274.7e6,
    "bf16_gemm_8192": 1173.7e6,      # profiles/gemm_tcgen05_pair_other_workloads.md
    "conv_fwd": 165.6e6,
    "conv_dedx": 165.1e6,
    "conv_dedw": 209.0e6,
    "fp8_bgemm_attn": 2154.3e6,
    "tf32_gemm_4096": 393.7e6,
    "fp32_gemm_4096": 1107.6e6,
    "compare_bf16": 2153.2e6,        # profiles/simt_helper_kernels.md
    "memory_write_add_f32": 3181.3e6,
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
    """Samples SM clocks, power and throttle reasons of one GPU with nvidia-smi, with time stamps, so that only the
    samples taken inside a timed window describe it."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index):
        self.proc, self.windows, self.samples = None, {}, None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "20"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def begin(self, name):
        self.windows[name] = [datetime.datetime.now(), None]

    def end(self, name):
        self.windows[name][1] = datetime.datetime.now()

    def _collect(self):
        if self.samples is not None:
            return
        self.samples = []
        if self.proc is None:
            return
        time.sleep(0.1)
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = ""
        for line in out.strip().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f")
                self.samples.append((ts, float(parts[1]), float(parts[2]), float(parts[3]),
                                     [nm for nm, val in zip(self.NAMES, parts[4:8]) if val.lower().startswith("active")]))
            except ValueError:
                continue

    def window(self, name, ms_per_step=None):
        """Clock record of the samples whose time stamp lies inside the window."""
        self._collect()
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples_under_load": 0}
        t0, t1 = self.windows[name]
        inside = [s for s in self.samples if t0 <= s[0] <= (t1 or t0)]
        mx = self.samples[-1][2] if self.samples else None
        rec = {"sm_mhz": statistics.median(s[1] for s in inside) if inside else None, "sm_max_mhz": mx,
               "power_w": statistics.median(s[3] for s in inside) if inside else None,
               "reasons": sorted({r for s in inside for r in s[4]}), "samples_under_load": len(inside),
               "window_s": ((t1 or t0) - t0).total_seconds()}
        if ms_per_step is not None and rec["sm_mhz"]:
            rec["ms_x_mhz"] = ms_per_step * rec["sm_mhz"]     # time x clock: compares runs taken at different clocks
        return rec

    def total(self):
        self._collect()
        return len(self.samples)


# ------------------------------------------------------------------------------------------ torch.distributed plumbing
def dist_setup():
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


# ------------------------------------------------------------------------------------------ one workload on one rank
class DeviceWorkload:
    """One configuration with this rank's operands resident in HBM, and `step()` = one launch of the hot path.

    strong scaling: the configuration is fixed and rank r holds rows / images [r, r+1) * total / world of it;
    weak scaling: every rank holds the whole per-GPU configuration. `gen` = "numpy" (the seeded host generators; kept
    for the end-to-end leg) or "device" (the library's tensor generator with the same distributions; no host copy).
    """

    def __init__(self, calc, name, rank, world, local, dist, scaling, gen="numpy", seed=1000):
        self.calc, self.name, self.wl = calc, name, WORKLOADS[name]
        self.rank, self.world, self.local, self.dist, self.scaling = rank, world, local, dist, scaling
        wl = self.wl
        self.bufs, self.host = [], None
        self.exchange = self.overlap = None
        strong = scaling == "strong" and world > 1
        if wl.get("exact"):
            calc.set_accumulation(abi.ACC_CHIP_EXACT)
        self.cast = abi.make_cast_params(abi.RM_NE) if wl["out_dtype"] != abi.FP32 else None
        if wl.get("stochastic"):
            self.cast = abi.make_cast_params(abi.RM_SR, clip_fp=True, rng_kind=abi.RNG_PHILOX, rng_seed=2024)
        elif wl.get("clip"):
            self.cast = abi.make_cast_params(abi.RM_NE, clip_fp=True)
        dev = abi.MEM_DEVICE
        if wl["kind"] == "gemm":
            b = wl.get("batch", 1)
            M, N, K = wl["M"], wl["N"], wl["K"]
            self.rows = M // world if strong else M
            assert not strong or (M % world == 0 and b == 1), "row sharding needs M divisible by the ranks"
            self.op = wl.get("op", abi.OP_AB)
            bd = [b] if b > 1 else []
            self.xs = [K, self.rows] + bd
            self.ws = ([K, N] if self.op == abi.OP_ABT else [N, K]) + bd
            self.os = [N, self.rows] + bd
            xb, wb = W.operand_biases(wl)
            self.kx = dict(fp_bias=xb, inf_nan_mode=W.inf_nan_mode(wl["in_dtype"]))
            self.kw = dict(fp_bias=wb, inf_nan_mode=W.inf_nan_mode(wl["w_dtype"]))
            self.ko = dict(fp_bias=7 if wl["out_dtype"] == abi.FP8_143 else 15, inf_nan_mode=W.inf_nan_mode(wl["out_dtype"]))
            nx, nw = int(np.prod(self.xs)), int(np.prod(self.ws))
            if gen == "numpy":
                # every rank draws the whole seeded configuration and keeps its rows: B is the same on all ranks
                x, w = W.synth_inputs(wl, seed=seed + (0 if strong else rank))
                if strong:
                    x = np.ascontiguousarray(x.reshape(M, K)[rank * self.rows:(rank + 1) * self.rows]).reshape(-1)
                self.host = (x, w)
                self.dx, self.dw = self._dev(x), self._dev(w)
            else:
                self.dx = self._alloc(nx * abi.ELEM_SIZE[wl["in_dtype"]])
                self.dw = self._alloc(nw * abi.ELEM_SIZE[wl["w_dtype"]])
                self._generate(self.dx, wl["in_dtype"], nx, self.kx, seed + 17 * rank)
                self._generate(self.dw, wl["w_dtype"], nw, self.kw, seed + 1)
            self.out_bytes = int(np.prod(self.os)) * abi.ELEM_SIZE[wl["out_dtype"]]
            self.dout = self._alloc(self.out_bytes)
            self.in_bytes = nx * abi.ELEM_SIZE[wl["in_dtype"]] + nw * abi.ELEM_SIZE[wl["w_dtype"]]
            self.flops_rank, self.alg_bytes_rank = W.workload_counts(wl, rows=self.rows)
            to, tx, tw = self.tensors(self.dx.ptr, self.dw.ptr, self.dout.ptr, dev)
            self.step = lambda: calc.do_batch_gemm(to, tx, tw, self.op, self.cast)
        else:
            self.images = CONV["B"] // world if strong else CONV["B"]
            assert not strong or CONV["B"] % world == 0
            xs, ws, ys = W.conv_shapes(wl, self.images)
            self.xs, self.ws, self.ys = xs, ws, ys
            s = wl.get("stride", 1)
            self.cp = abi.make_conv_params(2, (CONV["pad"], CONV["pad"]), (s, s), (1, 1))
            self.oshape = {abi.OP_FWD: ys, abi.OP_DEDX: xs, abi.OP_DEDW: ws}[wl["op"]]
            nx, nw, ny = int(np.prod(xs)), int(np.prod(ws)), int(np.prod(ys))
            if gen == "numpy":
                x, w, y = W.synth_inputs(wl, seed=seed + (0 if strong else rank))
                if strong:
                    per_x, per_y = nx // self.images, ny // self.images
                    x = x[rank * self.images * per_x:(rank + 1) * self.images * per_x]
                    y = y[rank * self.images * per_y:(rank + 1) * self.images * per_y]
                self.host = (x, w, y)
                self.dx, self.dw, self.dy = self._dev(x), self._dev(w), self._dev(y)
            else:
                self.dx, self.dw, self.dy = self._alloc(nx * 2), self._alloc(nw * 2), self._alloc(ny * 2)
                g = calc.generate
                g(T(self.dx.ptr, abi.BF16, [nx], mem_space=dev), abi.GEN_NORMAL, -1e30, 1e30, 0.0, 1.0, seed=seed + 17 * rank)
                g(T(self.dw.ptr, abi.BF16, [nw], mem_space=dev), abi.GEN_NORMAL, -1e30, 1e30, 0.0, float(np.sqrt(2.0 / (ws[1] * ws[2] * ws[3]))), seed=seed + 1)
                g(T(self.dy.ptr, abi.BF16, [ny], mem_space=dev), abi.GEN_NORMAL, -1e30, 1e30, 0.0, 0.01, seed=seed + 2 + 17 * rank)
            self.out_bytes = int(np.prod(self.oshape)) * abi.ELEM_SIZE[wl["out_dtype"]]
            self.dout = self._alloc(self.out_bytes)
            used = {abi.OP_FWD: (nx, nw), abi.OP_DEDX: (ny, nw), abi.OP_DEDW: (nx, ny)}[wl["op"]]
            self.in_bytes = 2 * sum(used)
            self.flops_rank, self.alg_bytes_rank = W.workload_counts(wl, images=self.images)
            to, tx, tw, ty = self.tensors(self.dx.ptr, self.dw.ptr, self.dy.ptr, self.dout.ptr, dev)
            op = wl["op"]
            if wl.get("fused_exchange"):
                from intel_gaudi3_software_b200.multi_gpu import PeerExchange
                self.exchange = PeerExchange(calc, int(np.prod(self.oshape)), dist, rank, world, deferred_output=True)
                self.step = lambda: self.exchange.dedw_allreduce(to, tx, tw, ty, self.cp)
            elif op == abi.OP_DEDW and dist is not None:
                self._setup_nccl_overlap(tx, tw, ty)
            else:
                self.step = lambda: calc.do_convolution(to, tx, tw, ty, self.cp, op, abi.RM_NE, self.cast)
        self.flops_job = self.flops_rank * world

    # ---- helpers
    def _alloc(self, nbytes):
        b = self.calc.alloc(nbytes)
        self.bufs.append(b)
        return b

    def _dev(self, array):
        b = self.calc.to_device(array)
        self.bufs.append(b)
        return b

    def _generate(self, buf, dtype, n, kw, seed):
        """The configuration's value distribution from the library's device generator (RandomSimTensorGenerator's role)."""
        t = T(buf.ptr, dtype, [n], mem_space=abi.MEM_DEVICE, **kw)
        if dtype in (abi.FP8_143, abi.FP8_152):
            # N(0,1) scaled so that amax (about 5.6 sigma over 10^8 draws) sits on the format's largest finite value
            top = (448.0 if dtype == abi.FP8_143 else 57344.0) * 2.0 ** ((7 if dtype == abi.FP8_143 else 15) - kw["fp_bias"])
            self.calc.generate(t, abi.GEN_NORMAL, -top, top, 0.0, top / 5.6, seed=seed)
        else:
            self.calc.generate(t, abi.GEN_UNIFORM, -1.0, 1.0, seed=seed)

    def tensors(self, *ptrs_and_space):
        wl = self.wl
        space = ptrs_and_space[-1]
        if wl["kind"] == "gemm":
            px, pw, po = ptrs_and_space[:3]
            return (T(po, wl["out_dtype"], self.os, mem_space=space, **self.ko), T(px, wl["in_dtype"], self.xs, mem_space=space, **self.kx),
                    T(pw, wl["w_dtype"], self.ws, mem_space=space, **self.kw))
        px, pw, py, po = ptrs_and_space[:4]
        return (T(po, wl["out_dtype"], self.oshape, mem_space=space), T(px, abi.BF16, self.xs, mem_space=space),
                T(pw, abi.BF16, self.ws, mem_space=space), T(py, abi.BF16, self.ys, mem_space=space))

    def _setup_nccl_overlap(self, tx, tw, ty):
        """dedw + NCCL: the fp32 partial dW is all-reduced on a second stream, double-buffered, so that the exchange of
        step i overlaps the convolution of step i+1 (as it would overlap the next layer's work in a training step)."""
        import torch
        calc, dist = self.calc, self.dist
        dev_t = torch.device("cuda", self.local)
        n = int(np.prod(self.oshape))
        bufs = [torch.empty(n, dtype=torch.float32, device=dev_t) for _ in range(2)]
        tos = [T(b.data_ptr(), abi.FP32, self.oshape, mem_space=abi.MEM_DEVICE) for b in bufs]
        comm = torch.cuda.Stream(device=dev_t)
        main = torch.cuda.current_stream(dev_t)
        calc.set_stream(main.cuda_stream)
        st = dict(i=0, done=[None, None])
        self.overlap = (st, main, bufs)

        def step():
            k = st["i"] & 1
            st["i"] += 1
            if st["done"][k] is not None:
                main.wait_event(st["done"][k])      # buffer k is free once its all-reduce finished
            calc.do_convolution(tos[k], tx, tw, ty, self.cp, abi.OP_DEDW, abi.RM_NE, None)
            ready = torch.cuda.Event()
            ready.record(main)
            with torch.cuda.stream(comm):
                comm.wait_event(ready)
                dist.all_reduce(bufs[k])
                ev = torch.cuda.Event()
                ev.record(comm)
            st["done"][k] = ev
        self.step = step

    def finish_exchanges(self):
        """The timed region ends when the last exchange has: order the NCCL stream's work before the stop mark."""
        if self.overlap is not None:
            st, main, _ = self.overlap
            for ev in st["done"]:
                if ev is not None:
                    main.wait_event(ev)

    def time_steps(self, steps, warmup):
        """ms for `steps` launches: CUDA events on the launching stream, barrier before, max over ranks after."""
        calc = self.calc
        for _ in range(warmup):
            self.step()
        self.finish_exchanges()
        calc.sync()
        barrier_and_max(self.dist, 0.0, self.local)
        calc.sync()
        calc.timer_start()
        for _ in range(steps):
            self.step()
        self.finish_exchanges()
        ms = calc.timer_stop()
        calc.sync()
        return barrier_and_max(self.dist, ms, self.local)

    def describe(self):
        wl = self.wl
        shape = {k: v for k, v in wl.items() if k in ("M", "N", "K", "batch")} or dict(CONV, stride=wl.get("stride", 1))
        out = {abi.BF16: "bf16", abi.FP8_143: "fp8_143", abi.FP32: "fp32"}[wl["out_dtype"]]
        out += "" if wl["out_dtype"] == abi.FP32 else (" stochastic rounding (Philox)" if wl.get("stochastic") else " RNE + clip" if wl.get("clip") else " RNE")
        return shape, out

    def close(self):
        if self.exchange is not None:
            self.exchange.close()
        if self.overlap is not None:
            self.calc.set_stream(None)
        for b in self.bufs:
            b.free()
        self.bufs = []


def config_dict(name, world, scaling):
    """The workload description both arms print (identical for --impl ours and --impl reference)."""
    wl = WORKLOADS[name]
    shape = {k: v for k, v in wl.items() if k in ("M", "N", "K", "batch")} or dict(CONV, stride=wl.get("stride", 1))
    out = {abi.BF16: "bf16", abi.FP8_143: "fp8_143", abi.FP32: "fp32"}[wl["out_dtype"]]
    out += "" if wl["out_dtype"] == abi.FP32 else (" stochastic rounding (Philox)" if wl.get("stochastic") else " RNE + clip" if wl.get("clip") else " RNE")
    if wl["kind"] == "conv" and wl["op"] == abi.OP_DEDW:
        shard = ("reduction (images) sharded; fp32 partials summed over NVLink inside the timed region by " +
                 ("the library's fused peer exchange" if wl.get("fused_exchange") else "an NCCL all-reduce (overlapped with the next step)"))
    else:
        shard = "rows of A / images sharded over the ranks, B / weights replicated, no collective"
    return {"workload": name, "shape": shape, "accumulate": "fp32", "output": out, "ranks": world,
            "scaling": scaling if world > 1 else "single GPU", "sharding": shard,
            "l2": "between steps nothing is flushed: operands + output exceed the 126 MB L2 at one GPU; shards that fit are marked in configs"}


def peak_for(wl, peaks, fp8_peak, sustained=False):
    """(peak TFLOP/s, note) of a tensor-bound workload."""
    bf16 = peaks["bf16_sustained"] if sustained else peaks["bf16"]
    kind = "sustained" if sustained else "burst"
    if wl["peak"] == "fp8":
        if fp8_peak and fp8_peak.get(kind):
            return fp8_peak[kind], "measured in this run: cuBLASLt e4m3 8192^3 -> bf16 (torch._scaled_mm), %s" % kind
        return 2.0 * bf16, "2 x the %s bf16 cuBLAS %s figure (fp8 GEMM could not be timed here: %s)" % (peaks["source"], kind, (fp8_peak or {}).get("error", "not run"))
    if wl["peak"] == "tf32":
        return bf16 / 2.0, "half the %s bf16 cuBLAS %s figure (tf32 runs at half the bf16 rate)" % (peaks["source"], kind)
    if wl["peak"] == "tf32x3":
        return bf16 / 6.0, "a sixth of the %s bf16 cuBLAS %s figure (fp32 operands: three tf32 products per pair, tf32 at half the bf16 rate)" % (peaks["source"], kind)
    return bf16, "%s bf16 cuBLAS %s figure" % (peaks["source"], kind)


def roofline_of(name, wl, flops, alg_bytes, ms_per_step, peaks, fp8_peak, sustained=False):
    if wl["bound"] == "tensor":
        peak, note = peak_for(wl, peaks, fp8_peak, sustained)
        achieved, unit = flops / (ms_per_step * 1e-3) / 1e12, "TFLOP/s"
    else:
        peak, note = peaks["hbm"], "%s HBM copy bandwidth" % peaks["source"]
        achieved, unit = alg_bytes / (ms_per_step * 1e-3) / 1e9, "GB/s"
    r = {"bound": wl["bound"], "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak,
         "traffic": NCU_TRAFFIC_BYTES.get(name), "peak_note": note,
         "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": alg_bytes}
    if wl["bound"] == "tensor" and wl["peak"] == "fp8":
        r["frac_of_2x_bf16"] = achieved / (2.0 * (peaks["bf16_sustained"] if sustained else peaks["bf16"]))
    return r


# ------------------------------------------------------------------------------------------ denominators measured here
def measure_fp8_peak(local, sampler=None):
    """A cuBLASLt e4m3 x e4m3 -> bf16 GEMM at 8192^3 with MEASURED_PEAKS.json's protocol: best of 10 (burst) and back to
    back for 4 s (sustained). A DENOMINATOR only: nothing on the product path calls it."""
    try:
        import torch
        dev = torch.device("cuda", local)
        n = 8192
        a = (torch.randn(n, n, device=dev) * 0.5).to(torch.float8_e4m3fn)
        b = (torch.randn(n, n, device=dev) * 0.5).to(torch.float8_e4m3fn).t()      # column-major, as cuBLASLt wants B
        one = torch.tensor(1.0, device=dev)

        def mm():
            return torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
        for _ in range(3):
            mm()
        torch.cuda.synchronize(dev)
        best = 1e9
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            mm()
            e1.record()
            e1.synchronize()
            best = min(best, e0.elapsed_time(e1))
        flops = 2.0 * n ** 3
        if sampler:
            sampler.begin("fp8_peak")
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        reps, t0 = 0, time.perf_counter()
        e0.record()
        while time.perf_counter() - t0 < 4.0:
            for _ in range(50):
                mm()
            reps += 50
            torch.cuda.synchronize(dev)
        e1.record()
        e1.synchronize()
        if sampler:
            sampler.end("fp8_peak")
        sustained_ms = e0.elapsed_time(e1) / reps
        return {"burst": flops / (best * 1e-3) / 1e12, "sustained": flops / (sustained_ms * 1e-3) / 1e12, "how":
                "torch._scaled_mm e4m3 8192^3 -> bf16: best of 10 (burst), back to back for 4 s (sustained)"}
    except Exception as exc:   # the denominator is optional; the note then says which stand-in was used
        return {"error": "%s: %s" % (type(exc).__name__, str(exc)[:120])}


def measure_copy_bandwidth(local, nbytes=256 << 20):
    """Pinned host <-> device copy bandwidth of this box, GB/s: each direction alone and both at once (the end-to-end
    leg's roofline). Best of three."""
    try:
        import torch
        dev = torch.device("cuda", local)
        h_in = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        h_out = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        d_in, d_out = torch.empty(nbytes, dtype=torch.uint8, device=dev), torch.empty(nbytes, dtype=torch.uint8, device=dev)
        s1, s2 = torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def run(up, down):
            best = 1e9
            for _ in range(4):
                torch.cuda.synchronize(dev)
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                s1.wait_event(e0)
                s2.wait_event(e0)
                if up:
                    with torch.cuda.stream(s1):
                        d_in.copy_(h_in, non_blocking=True)
                if down:
                    with torch.cuda.stream(s2):
                        h_out.copy_(d_out, non_blocking=True)
                torch.cuda.current_stream(dev).wait_stream(s1)
                torch.cuda.current_stream(dev).wait_stream(s2)
                e1.record()
                e1.synchronize()
                best = min(best, e0.elapsed_time(e1))
            return (int(up) + int(down)) * nbytes / (best * 1e-3) / 1e9
        return {"h2d_gbs": run(True, False), "d2h_gbs": run(False, True), "both_gbs": run(True, True),
                "how": "pinned 256 MiB copies, cudaMemcpyAsync on two streams, best of 4"}
    except Exception as exc:
        return {"error": "%s: %s" % (type(exc).__name__, str(exc)[:120])}


# ------------------------------------------------------------------------------------------ HBM-bound helper kernels
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
    sampler.begin("timed")
    calc.timer_start()
    for _ in range(steps):
        step()
    ms = calc.timer_stop() / steps
    sampler.end("timed")
    clocks = sampler.window("timed", ms)
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


# ------------------------------------------------------------------------------------------ our arm
def end_to_end(calc, dw, lib, dist, rank, world, local, steps):
    """The same metric through the public API with pinned host buffers: every step copies the step's inputs host ->
    device and its result device -> host inside the timed region. One GPU: the C ABI call with host tensors (the library
    pipelines row blocks of A and of the output around the GEMM). Several GPUs: the multi-GPU driver's host-tensor GEMM
    (each rank uploads its rows of A and 1/N of B, B is spread over NVLink, outputs go back per rank)."""
    wl = dw.wl

    def pinned(nbytes):
        p = C.c_void_p()
        assert lib.mmeb200_host_alloc(C.byref(p), nbytes) == 0
        return p.value
    hp = []
    for h in dw.host:
        p = pinned(h.nbytes)
        C.memmove(p, h.ctypes.data, h.nbytes)
        hp.append(p)
    hout = pinned(dw.out_bytes)
    h2d = dw.in_bytes
    if wl["kind"] == "gemm":
        eo, ex, ew = dw.tensors(hp[0], hp[1], hout, abi.MEM_HOST)
        if world > 1 and dw.scaling == "strong":
            from intel_gaudi3_software_b200.multi_gpu import ShardedCalculator
            sc = ShardedCalculator(calc, dist, rank, world, device=local)
            step = lambda: sc.host_gemm_shared_b(eo, ex, ew, dw.op, dw.cast)   # noqa: E731
            nw = int(np.prod(dw.ws)) * abi.ELEM_SIZE[wl["w_dtype"]]
            h2d = dw.in_bytes - nw + nw // world                                   # this rank's PCIe bytes; the rest of B arrives over NVLink
        else:
            step = lambda: calc.do_batch_gemm(eo, ex, ew, dw.op, dw.cast)          # noqa: E731
    else:
        eo, ex, ew, ey = dw.tensors(hp[0], hp[1], hp[2], hout, abi.MEM_HOST)
        if dw.exchange is not None:
            step = lambda: dw.exchange.dedw_allreduce(eo, ex, ew, ey, dw.cp)       # noqa: E731
        elif wl["op"] == abi.OP_DEDW and dist is not None:
            import torch
            calc.set_stream(None)
            n = int(np.prod(dw.oshape))
            part = torch.empty(n, dtype=torch.float32, device=torch.device("cuda", local))
            tp = T(part.data_ptr(), abi.FP32, dw.oshape, mem_space=abi.MEM_DEVICE)
            host_t = torch.frombuffer((C.c_uint8 * dw.out_bytes).from_address(hout), dtype=torch.float32)

            def step():
                calc.do_convolution(tp, ex, ew, ey, dw.cp, abi.OP_DEDW, abi.RM_NE, None)
                calc.sync()
                dist.all_reduce(part)
                host_t.copy_(part)
        else:
            step = lambda: calc.do_convolution(eo, ex, ew, ey, dw.cp, wl["op"], abi.RM_NE, dw.cast)  # noqa: E731
    for _ in range(2):   # the first host-tensor calls size the library's staging arena
        step()
    calc.sync()
    barrier_and_max(dist, 0.0, local)
    t0 = time.perf_counter()
    calc.timer_start()
    for _ in range(steps):
        step()
    ms = calc.timer_stop() / steps
    wall_ms = (time.perf_counter() - t0) * 1e3 / steps
    ms = max(ms, wall_ms) if world > 1 and wl["kind"] == "gemm" else ms      # the driver path spans several streams: the host clock bounds it
    ms = barrier_and_max(dist, ms, local)
    checksum = int(np.frombuffer((C.c_uint8 * min(dw.out_bytes, 4096)).from_address(hout), dtype=np.uint8).sum())
    return {"value": dw.flops_job / (ms * 1e-3) / 1e12, "unit": "TFLOP/s", "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(dw.out_bytes), "ms_per_step": ms, "result_checksum": checksum,
            "bytes_are": "per rank" if world > 1 else "whole job"}


def run_ours(args):
    import intel_gaudi3_software_b200 as pkg
    wl = WORKLOADS[args.workload]
    if wl["kind"] == "stream":
        return run_stream(args)
    rank, world, local, dist = dist_setup()
    scaling = args.scaling if world > 1 else "strong"
    calc = pkg.Calculator(device=local)
    lib = calc.lib
    peaks = measured_peaks()
    warmup = max(args.warmup, 3)

    # ---- headline: device-resident timing of exactly `steps` launches
    dw = DeviceWorkload(calc, args.workload, rank, world, local, dist, scaling, gen="numpy")
    sampler = ClockSampler(local) if rank == 0 else None
    launches0 = calc.launch_count()
    dw.time_steps(1, warmup)                       # warm-up (and one untimed launch behind a barrier)
    launches0 = calc.launch_count()
    if sampler:
        sampler.begin("timed")
    ms = dw.time_steps(args.steps, 0)
    if sampler:
        sampler.end("timed")
    launches = calc.launch_count() - launches0
    ms_per_step = ms / args.steps
    value = dw.flops_job / (ms_per_step * 1e-3) / 1e12

    # ---- the same launch back to back for >= sustain seconds, clocks sampled inside the window
    sustained = None
    if args.sustain > 0:
        n_sus = max(args.steps, int(args.sustain * 1e3 / max(ms_per_step, 1e-3)) + 1)
        if sampler:
            sampler.begin("sustained")
        sus_ms = dw.time_steps(n_sus, 0) / n_sus
        if sampler:
            sampler.end("sustained")
        sustained = {"value": dw.flops_job / (sus_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "steps": n_sus, "ms_per_step": sus_ms}

    # ---- end to end through the public API with pinned host buffers
    e2e = end_to_end(calc, dw, lib, dist, rank, world, local, max(3, min(args.steps, 10)))
    dw.close()

    # ---- every benchmark configuration, device-resident, inputs from the library's generator
    configs = {}
    names = [] if args.configs == "none" else (DEFAULT_CONFIGS if world == 1 else MULTI_GPU_CONFIGS)
    cfg_raw = {}
    for name in names:
        try:
            cw = DeviceWorkload(calc, name, rank, world, local, dist, scaling, gen="device")
            steps_c = 20 if cw.flops_rank < 2e12 else 10
            time.sleep(0.5)     # start every configuration from the idle state the headline starts from, not from the heat of the one before
            cw.time_steps(1, 3)
            l0 = calc.launch_count()
            c_ms = cw.time_steps(steps_c, 0) / steps_c
            cfg_raw[name] = (cw.flops_job, cw.flops_rank, cw.alg_bytes_rank, c_ms, steps_c, (calc.launch_count() - l0) / steps_c,
                             cw.in_bytes + cw.out_bytes)
            cw.close()
        except Exception as exc:   # a configuration that cannot run is reported, not hidden
            cfg_raw[name] = "%s: %s" % (type(exc).__name__, str(exc)[:160])

    # ---- denominators measured in this run (never on the product path): fp8 tensor peak, pinned copy bandwidth
    fp8_peak = copy_bw = None
    if rank == 0 and not args.skip_peaks:
        calc.sync()
        copy_bw = measure_copy_bandwidth(local)
        fp8_peak = measure_fp8_peak(local, sampler)

    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        calc.close()
        return

    for name, raw in cfg_raw.items():
        if isinstance(raw, str):
            configs[name] = {"error": raw}
            continue
        flops_job, flops_rank, alg_rank, c_ms, steps_c, launches_c, footprint = raw
        cwl = WORKLOADS[name]
        r = roofline_of(name, cwl, flops_rank, alg_rank, c_ms, peaks, fp8_peak)
        configs[name] = {"value": flops_job / (c_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": c_ms, "steps": steps_c,
                         "launches_per_step": launches_c, "frac": r["frac"], "bound": r["bound"], "achieved_per_gpu": r["achieved"],
                         "roofline_unit": r["unit"], "peak": r["peak"], "peak_note": r["peak_note"], "traffic": r["traffic"] if world == 1 else None,
                         "fits_l2": bool(footprint <= L2_BYTES)}
        if "frac_of_2x_bf16" in r:
            configs[name]["frac_of_2x_bf16"] = r["frac_of_2x_bf16"]

    roof = roofline_of(args.workload, wl, dw.flops_rank, dw.alg_bytes_rank, ms_per_step, peaks, fp8_peak)
    if world > 1:
        roof["traffic"] = None      # the captures were taken on the one-GPU shape
    clocks = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0, "samples_under_load": 0}
    if sampler:
        timed = sampler.window("timed", ms_per_step)
        sus = sampler.window("sustained", sustained["ms_per_step"]) if sustained else None
        under = sus if (sus and sus["samples_under_load"]) else timed
        clocks = {"sm_mhz": under["sm_mhz"], "sm_max_mhz": under["sm_max_mhz"], "reasons": sorted(set(timed["reasons"]) | set((sus or timed)["reasons"])),
                  "samples": sampler.total(), "samples_under_load": timed["samples_under_load"] + (sus["samples_under_load"] if sus else 0),
                  "window": "the %d timed steps last %.1f ms, shorter than the 20 ms sampling period: sm_mhz is the median inside the sustained run "
                            "of the same launch that follows them" % (args.steps, ms) if under is sus else "samples inside the timed steps",
                  "timed_steps": timed, "sustained": sus}
        if fp8_peak and "error" not in fp8_peak:
            fp8_peak["clocks"] = sampler.window("fp8_peak")
    if sustained:
        sroof = roofline_of(args.workload, wl, dw.flops_rank, dw.alg_bytes_rank, sustained["ms_per_step"], peaks, fp8_peak, sustained=True)
        sustained.update({"frac": sroof["frac"], "peak": sroof["peak"], "peak_note": sroof["peak_note"]})
        if "frac_of_2x_bf16" in sroof:
            sustained["frac_of_2x_bf16"] = sroof["frac_of_2x_bf16"]
    if copy_bw and "error" not in copy_bw:
        moved = e2e["h2d_bytes_per_step"] + e2e["d2h_bytes_per_step"]
        ach = moved / (e2e["ms_per_step"] * 1e-3) / 1e9
        e2e["roofline"] = {"bound": "host<->device copies", "achieved": ach, "peak": copy_bw["both_gbs"], "unit": "GB/s",
                           "frac": ach / copy_bw["both_gbs"], "peak_note": "pinned H2D + D2H at once, measured in this run on this rank's GPU",
                           "h2d_alone_gbs": copy_bw["h2d_gbs"], "d2h_alone_gbs": copy_bw["d2h_gbs"]}
    elif copy_bw:
        e2e["roofline"] = copy_bw
    line = {
        "metric": "GEMM/conv TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": args.scaling,   # the N = 1 line of a strong-scaling series says so too
        "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": config_dict(args.workload, world, scaling),
        "e2e": e2e, "gpu_launches": launches, "clocks": clocks, "roofline": roof, "sustained": sustained, "configs": configs,
        "configs_protocol": "each configuration starts after 0.5 s of idle like the headline: 4 warm-up steps, then 10 or 20 timed steps",
        "measured_peaks": {"bf16_tflops": peaks["bf16"], "bf16_tflops_sustained": peaks["bf16_sustained"], "hbm_gbs": peaks["hbm"],
                           "source": peaks["source"], "fp8": fp8_peak, "host_copy": copy_bw},
    }
    if world == 1 and not args.skip_cpu_baseline:
        line["cpu_baseline"] = cpu_baseline(wl, args.workload, budget_s=12.0)
    print(json.dumps(line))
    calc.close()


# ------------------------------------------------------------------------------------------ the reference's CPU calculator
_CPU_W_CACHE = {}


def cpu_sample(wl, rows_hint=None):
    """The CPU calculator (the compiled reference when present, else the C restatement) and the host threads it uses."""
    from oracle import Port, Ref, have_ref
    lib = Ref() if have_ref() else Port()
    threads = lib.hardware_threads()
    return lib, threads


def cpu_run(lib, wl, rows, threads, seed=1000):
    """One bounded CPU sample; returns (seconds, flops)."""
    if wl["kind"] == "gemm":
        N, K = wl["N"], wl["K"]
        key = (wl["w_dtype"], N, K, seed)
        if key not in _CPU_W_CACHE:   # B is the same for every sample of a run: draw it once
            r = np.random.default_rng(seed + 1)
            _CPU_W_CACHE[key] = (W.f32_to_bf16_rne(r.uniform(-1, 1, K * N).astype(np.float32)) if wl["w_dtype"] == abi.BF16
                                 else W.quantise_fp8(r.standard_normal(K * N, dtype=np.float32), wl["w_dtype"], 7))
        w = _CPU_W_CACHE[key]
        r = np.random.default_rng(seed)
        x = (W.f32_to_bf16_rne(r.uniform(-1, 1, rows * K).astype(np.float32)) if wl["in_dtype"] == abi.BF16
             else W.quantise_fp8(r.standard_normal(rows * K, dtype=np.float32), wl["in_dtype"], 7))
        x_bias, w_bias = W.operand_biases(wl)
        acc = np.zeros(rows * N, np.float32)
        # the CPU sample uses the 'ab' orientation; the arithmetic per output is the same
        tx = T(x, wl["in_dtype"], [K, rows], fp_bias=x_bias, inf_nan_mode=W.inf_nan_mode(wl["in_dtype"]))
        tw = T(w, wl["w_dtype"], [N, K], fp_bias=w_bias, inf_nan_mode=W.inf_nan_mode(wl["w_dtype"]))
        t0 = time.perf_counter()
        rc = lib.bgemm(T(acc, abi.FP32, [N, rows]), tx, tw, abi.OP_AB, threads=threads)
        assert rc == 0
        if wl["out_dtype"] != abi.FP32:
            lib.fp32_to_bf16(acc)
        dt = time.perf_counter() - t0
        return dt, 2.0 * rows * N * K
    # convolution: whole-width strips of one image (`rows` output rows of the 56-wide grid)
    c = dict(CONV, B=1, H=rows, W=CONV["W"])
    xs, ws, ys = [c["C"], c["W"], c["H"], 1], [c["K"], c["C"], c["S"], c["R"]], [c["K"], c["W"], c["H"], 1]
    rng = np.random.default_rng(seed)
    x = W.f32_to_bf16_rne(rng.standard_normal(int(np.prod(xs)), dtype=np.float32))
    w = W.f32_to_bf16_rne(rng.standard_normal(int(np.prod(ws)), dtype=np.float32) * np.float32(0.0295))
    y = W.f32_to_bf16_rne(rng.standard_normal(int(np.prod(ys)), dtype=np.float32) * np.float32(0.01))
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


def sample_text(wl, rows):
    return ("%d rows of A x all of B (K whole)" % rows) if wl["kind"] == "gemm" else ("one image of %d x %d pixels" % (rows, CONV["W"]))


def cpu_baseline(wl, name, budget_s):
    lib, threads = cpu_sample(wl)
    rows = pick_rows(lib, wl, threads, budget_s)
    dt, fl = cpu_run(lib, wl, rows, threads)
    return {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": lib.kind, "sample": sample_text(wl, rows), "seconds": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    wl = WORKLOADS[args.workload]
    if wl["kind"] == "stream":
        print(json.dumps({"impl": "reference", "unavailable": "the helper-kernel workloads have no CPU arm in this benchmark"}))
        return
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
    scaling = args.scaling if world > 1 else "strong"
    line = {
        "impl": "reference", "metric": "GEMM/conv TFLOP/s", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": t / args.steps * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": wl["dtype"], "data": "synthetic",
        "config": config_dict(args.workload, world, scaling),
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": lib.kind, "sample": sample_text(wl, rows),
                         "note": "the reference's CPU calculator on the host cores; each step is a bounded sample of the workload, "
                                 "so the figure is a rate, not the time of the whole configuration"},
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
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: split the fixed configuration over the ranks (strong) or give every rank the whole of it (weak)")
    ap.add_argument("--configs", default="default", choices=["default", "none"], help="also time every benchmark configuration")
    ap.add_argument("--sustain", type=float, default=2.0, help="seconds of the back-to-back run (0 = skip)")
    ap.add_argument("--skip-cpu-baseline", action="store_true", help="leave the CPU baseline leg out (sweeps)")
    ap.add_argument("--skip-peaks", action="store_true", help="do not time the fp8 cuBLASLt GEMM / host copies (sweeps)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
