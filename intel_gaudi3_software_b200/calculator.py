"""Host-side handle on libmme_b200.so with the reference calculator's method names.

The reference's calculator is a C++ class (CPUCalculator, mme/mme_reference/mme_reference.h:108-191);
its C++ drop-in lives in intel_gaudi3_software_b200/cpp. This Python class exposes the same
operations over the same C ABI for the tests, the benchmark and the multi-GPU driver. Every method
raises MmeError (the counterpart of MME_ASSERT -> MMEStackException, mme/include/mme_assert.h:27-60)
when the library reports a failure. Nothing here computes on the CPU.
"""
import ctypes as C

import numpy as np

from . import abi


class MmeError(RuntimeError):
    def __init__(self, status, message):
        super().__init__("mme_b200 status %d: %s" % (status, message))
        self.status = status


class DeviceBuffer:
    """A device allocation owned by a Calculator (freed with it or by free())."""

    def __init__(self, calc, nbytes):
        self.calc, self.nbytes = calc, nbytes
        p = C.c_void_p()
        calc._check(calc.lib.mmeb200_malloc(calc.ctx, C.byref(p), nbytes))
        self.ptr = p.value

    def upload(self, array):
        a = np.ascontiguousarray(array)
        assert a.nbytes <= self.nbytes
        self.calc._check(self.calc.lib.mmeb200_memcpy_h2d(self.calc.ctx, self.ptr, a.ctypes.data, a.nbytes))
        return self

    def download(self, dtype, count=None):
        dt = np.dtype(dtype)
        n = self.nbytes // dt.itemsize if count is None else count
        out = np.empty(n, dtype=dt)
        self.calc._check(self.calc.lib.mmeb200_memcpy_d2h(self.calc.ctx, out.ctypes.data, self.ptr, out.nbytes))
        return out

    def free(self):
        if self.ptr:
            self.calc.lib.mmeb200_free(self.calc.ctx, self.ptr)
            self.ptr = None


class Calculator:
    """CPUCalculator(chip, ..., seed, lfsrNumRegs, lfsr, polynomial) on one B200."""

    def __init__(self, chip=abi.CHIP_GAUDI3, device=0, seed=0, lfsr_num_regs=256, lfsr=None, polynomial=0, accumulation=abi.ACC_TENSOR_CORE):
        self.lib = abi.load_library()
        ctx = C.c_void_p()
        regs = None
        if lfsr is not None:
            arr = np.ascontiguousarray(lfsr, dtype=np.uint32)
            lfsr_num_regs = arr.size
            regs = arr.ctypes.data_as(C.POINTER(C.c_uint32))
        rc = self.lib.mmeb200_create(C.byref(ctx), chip, device, seed, lfsr_num_regs, regs, polynomial)
        if rc != 0:
            raise MmeError(rc, "mmeb200_create failed (no B200 visible?)" if rc == abi.ERR_NO_DEVICE else "mmeb200_create failed")
        self.ctx = ctx
        self.device = device
        if accumulation != abi.ACC_TENSOR_CORE:
            self.set_accumulation(accumulation)

    def close(self):
        if getattr(self, "ctx", None):
            self.lib.mmeb200_destroy(self.ctx)
            self.ctx = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, rc):
        if rc != 0:
            raise MmeError(rc, self.lib.mmeb200_last_error(self.ctx).decode())

    # ---- the calculator's operations -----------------------------------------------------
    def limit_num_of_threads(self, n):
        self._check(self.lib.mmeb200_limit_num_of_threads(self.ctx, n))

    def do_batch_gemm(self, out, x, w, op, cast=None):
        self._check(self.lib.mmeb200_bgemm(self.ctx, out, x, w, op, cast))

    def do_convolution(self, out, x, w, y, params, op, rm=abi.RM_NE, cast=None):
        self._check(self.lib.mmeb200_conv(self.ctx, out, x, w, y, params, op, rm, cast))

    def do_activation(self, out, acc, cast):
        self._check(self.lib.mmeb200_activation(self.ctx, out, acc, cast))

    def do_memory_write(self, mem, mme_out, reduction_op=abi.RED_NONE, reduction_rm=0, clip_fp=False):
        self._check(self.lib.mmeb200_memory_write(self.ctx, mem, mme_out, reduction_op, reduction_rm, int(clip_fp)))

    def do_dma(self, out, x, op):
        self._check(self.lib.mmeb200_dma(self.ctx, out, x, op))

    def convert(self, out, inp, cast=None):
        self._check(self.lib.mmeb200_convert(self.ctx, out, inp, cast))

    def compare(self, a, b, cd_size, num_partials=1, bit_exact=False):
        """TensorComparator::doCompare / doCompareBitExact on the device: (mismatching elements, lowest mismatching index)."""
        r = abi.CompareResult()
        self._check(self.lib.mmeb200_compare(self.ctx, a, b, cd_size, num_partials, int(bit_exact), C.byref(r)))
        return int(r.mismatches), int(r.first_index)

    def set_accumulation(self, mode):
        """abi.ACC_TENSOR_CORE (default) or abi.ACC_CHIP_EXACT (accumulators bit-identical to the reference's Gaudi3 model)."""
        self._check(self.lib.mmeb200_set_accumulation(self.ctx, mode))

    def generate(self, out, kind, min_value=0.0, max_value=0.0, mean=0.0, std_dev=0.0, seed=0, packing=0, level=0):
        """RandomSimTensorGenerator on the device: fills `out` (uniform / normal / fill / unit / reduction packing)."""
        g = abi.GenerateParams(kind, min_value, max_value, mean, std_dev, packing, level, seed)
        self._check(self.lib.mmeb200_generate(self.ctx, out, C.byref(g)))

    def peer_alloc(self, nbytes):
        """Zero-filled device memory that other processes can map: returns (device pointer, 64-byte handle)."""
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        self._check(self.lib.mmeb200_peer_alloc(self.ctx, nbytes, C.byref(ptr), handle))
        return ptr.value, handle.raw

    def peer_open(self, handle):
        ptr = C.c_void_p()
        self._check(self.lib.mmeb200_peer_open(self.ctx, handle, C.byref(ptr)))
        return ptr.value

    def peer_close(self, ptr):
        self._check(self.lib.mmeb200_peer_close(self.ctx, ptr))

    def do_convolution_dedw_allreduce(self, out, x, w, y, params, group):
        self._check(self.lib.mmeb200_conv_dedw_allreduce(self.ctx, out, x, w, y, params, group))

    def gemm_splitk_static(self, out, x, w, op, splits):
        """Split-K GEMM whose partial sums live in the library's fixed 16 MiB device array: for callers
        that may not allocate (see include/mme_b200.h). Device tensors only."""
        self._check(self.lib.mmeb200_gemm_splitk_static(self.ctx, out, x, w, op, splits))

    # ---- state and plumbing -----------------------------------------------------------------
    def get_lfsr(self, n=256):
        regs = np.zeros(n, dtype=np.uint32)
        poly = C.c_uint32()
        self._check(self.lib.mmeb200_get_lfsr(self.ctx, regs.ctypes.data_as(C.POINTER(C.c_uint32)), n, C.byref(poly)))
        return regs, poly.value

    def set_lfsr(self, regs, polynomial=0):
        arr = np.ascontiguousarray(regs, dtype=np.uint32)
        self._check(self.lib.mmeb200_set_lfsr(self.ctx, arr.ctypes.data_as(C.POINTER(C.c_uint32)), arr.size, polynomial))

    def set_option(self, name, value):
        """Force one of the planner's choices (include/mme_b200.h: mmeb200_set_option); value < 0 = automatic."""
        self._check(self.lib.mmeb200_set_option(self.ctx, name.encode(), int(value)))

    def set_stream(self, cuda_stream_handle):
        self._check(self.lib.mmeb200_set_stream(self.ctx, cuda_stream_handle))

    def sync(self, timeout_ns=0):
        self._check(self.lib.mmeb200_sync(self.ctx, timeout_ns))

    def alloc(self, nbytes):
        return DeviceBuffer(self, nbytes)

    def to_device(self, array):
        a = np.ascontiguousarray(array)
        return DeviceBuffer(self, max(a.nbytes, 16)).upload(a)

    def timer_start(self):
        self._check(self.lib.mmeb200_timer_start(self.ctx))

    def timer_stop(self):
        ms = C.c_float()
        self._check(self.lib.mmeb200_timer_stop(self.ctx, C.byref(ms)))
        return ms.value

    def mem_info(self):
        """(free, total) bytes of device memory on the calculator's GPU."""
        free, total = C.c_size_t(), C.c_size_t()
        self._check(self.lib.mmeb200_mem_info(self.ctx, C.byref(free), C.byref(total)))
        return free.value, total.value

    def launch_count(self):
        return int(self.lib.mmeb200_launch_count(self.ctx))
