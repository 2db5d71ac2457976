"""ctypes image of include/mme_b200.h: enums, plain-data structs and the library loader.

This module is plumbing for the tests, the benchmark and the multi-GPU driver; the product is the
shared library it loads. There is no CPU path: if the library is missing, loading raises.
"""
import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "lib", "libmme_b200.so")

# EMmeDataType values (mme/include/mme_common/mme_common_enum.h:32-62)
FP8_143, FP8_152, FP16, BF16, FP32, FP32_IEEE, TF32 = 9, 10, 11, 12, 13, 14, 15
# EMmeOpType values (mme_common_enum.h:83-102)
OP_FWD, OP_DEDX, OP_DEDW, OP_DET_DEDW, OP_TRANSPOSED_DEDX = 0, 1, 2, 3, 4
OP_AB, OP_ABT, OP_ATB, OP_ATBT = 5, 6, 7, 8
OP_GEMM_TRANSPOSE, OP_MEMCPY, OP_TRANS, OP_REDUCTION_ADD = 9, 10, 11, 12
# RoundingMode values (mme_common_enum.h:67-81)
RM_NE, RM_Z, RM_UP, RM_DOWN, RM_SR, RM_HAZ, RM_SR_NE_DNORM = 0, 1, 2, 3, 4, 6, 7
# InfNanMode (mme_common_enum.h:191-197)
INFNAN_FULL, INFNAN_NONE, INFNAN_MINIMAL = 0, 1, 2
# EMmeReductionOp (mme_common_enum.h:321-332)
RED_ADD, RED_SUB, RED_MIN, RED_MAX, RED_MAX_0, RED_NONE = 0, 1, 2, 3, 4, 5
CHIP_GAUDI, CHIP_GAUDI2, CHIP_GAUDI3 = 0, 1, 2
MEM_HOST, MEM_DEVICE = 0, 1
RNG_LFSR, RNG_PHILOX = 0, 1

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_TIMEOUT, ERR_NO_DEVICE, ERR_DEVICE_WAIT = 0, -1, -2, -3, -4, -5, -6

ELEM_SIZE = {FP8_143: 1, FP8_152: 1, BF16: 2, FP16: 2, FP32: 4, FP32_IEEE: 4, TF32: 4}
NP_DTYPE = {FP8_143: np.uint8, FP8_152: np.uint8, BF16: np.uint16, FP16: np.uint16, FP32: np.float32,
            FP32_IEEE: np.float32, TF32: np.float32}


class Tensor(C.Structure):
    """mmeb200_tensor: plain-data image of MmeSimTensor (mme/mme_reference/sim_tensor.h:9-52)."""
    _fields_ = [("dtype", C.c_int32), ("dims", C.c_int32), ("sizes", C.c_uint32 * 5), ("strides", C.c_uint32 * 5),
                ("fp_bias", C.c_uint32), ("inf_nan_mode", C.c_int32), ("mem_space", C.c_int32),
                ("reserved", C.c_int32), ("data", C.c_void_p)]


class ConvParams(C.Structure):
    """mmeb200_conv_params: ConvolutionParams (mme/mme_reference/convolution_params.h:7-29)."""
    _fields_ = [("dim", C.c_int32), ("padding", C.c_int32 * 4), ("stride", C.c_int32 * 4),
                ("dilation", C.c_int32 * 4), ("padding_value", C.c_uint32), ("relu", C.c_int32)]


class CastParams(C.Structure):
    """mmeb200_cast_params: the cast arguments of doActivation (mme/mme_reference/mme_reference.h:162-172)."""
    _fields_ = [("rounding", C.c_int32), ("relu", C.c_int32), ("clip_fp", C.c_int32), ("clip_inf_in", C.c_int32),
                ("flush_denorms", C.c_int32), ("stochastic_ftz_fp8", C.c_int32), ("rng_kind", C.c_int32),
                ("reserved", C.c_int32), ("rng_seed", C.c_uint64), ("rng_offset", C.c_uint64)]


class PeerGroup(C.Structure):
    """mmeb200_peer_group: exchange buffers and flag blocks of the ranks taking part in a fused dedw exchange."""
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("slots", C.c_void_p * 8), ("flags", C.c_void_p * 8),
                ("step", C.c_uint32), ("deferred_output", C.c_uint32)]


class CompareResult(C.Structure):
    """mmeb200_compare_result."""
    _fields_ = [("mismatches", C.c_uint64), ("first_index", C.c_uint64)]


class GenerateParams(C.Structure):
    """mmeb200_generate_params."""
    _fields_ = [("kind", C.c_int32), ("min_value", C.c_float), ("max_value", C.c_float), ("mean", C.c_float), ("std_dev", C.c_float),
                ("packing", C.c_uint32), ("level", C.c_uint32), ("seed", C.c_uint64)]


ACC_TENSOR_CORE, ACC_CHIP_EXACT = 0, 1
GEN_UNIFORM, GEN_NORMAL, GEN_FILL, GEN_UNIT, GEN_REDUCTION_PACKING = 0, 1, 2, 3, 4


def dense_strides(sizes):
    s, acc = [], 1
    for n in sizes:
        s.append(acc)
        acc *= n
    return s


def make_tensor(data, dtype, sizes, strides=None, fp_bias=0, inf_nan_mode=INFNAN_FULL, mem_space=MEM_HOST):
    """Build a Tensor over `data` (a numpy array, kept alive by the caller, or a raw address).

    sizes[0] is the fastest dimension, as in the reference.
    """
    sizes = list(sizes)
    dims = len(sizes)
    sizes5 = sizes + [1] * (5 - dims)
    if strides is None:
        strides5 = dense_strides(sizes5)
    else:
        strides = list(strides)
        strides5 = strides + [0] * (5 - len(strides))
        acc = strides5[dims - 1] * sizes5[dims - 1] if dims else 1
        for d in range(dims, 5):
            strides5[d] = acc
    t = Tensor()
    t.dtype, t.dims = dtype, dims
    t.sizes = (C.c_uint32 * 5)(*sizes5)
    t.strides = (C.c_uint32 * 5)(*strides5)
    t.fp_bias, t.inf_nan_mode, t.mem_space, t.reserved = fp_bias, inf_nan_mode, mem_space, 0
    if isinstance(data, np.ndarray):
        t.data = data.ctypes.data
        t._keep = data
    else:
        t.data = int(data) if data is not None else None
    return t


def make_conv_params(dim=2, padding=(0, 0, 0, 0), stride=(1, 1, 1, 1), dilation=(1, 1, 1, 1), relu=False):
    p = ConvParams()
    p.dim = dim
    pad4 = list(padding) + [0] * (4 - len(padding))
    st4 = list(stride) + [1] * (4 - len(stride))
    dl4 = list(dilation) + [1] * (4 - len(dilation))
    p.padding = (C.c_int32 * 4)(*pad4)
    p.stride = (C.c_int32 * 4)(*st4)
    p.dilation = (C.c_int32 * 4)(*dl4)
    p.padding_value, p.relu = 0, int(relu)
    return p


def make_cast_params(rounding=RM_NE, relu=False, clip_fp=False, clip_inf_in=False, flush_denorms=False,
                     stochastic_ftz_fp8=False, rng_kind=RNG_LFSR, rng_seed=0, rng_offset=0):
    c = CastParams()
    c.rounding, c.relu, c.clip_fp, c.clip_inf_in = rounding, int(relu), int(clip_fp), int(clip_inf_in)
    c.flush_denorms, c.stochastic_ftz_fp8, c.rng_kind, c.reserved = int(flush_denorms), int(stochastic_ftz_fp8), rng_kind, 0
    c.rng_seed, c.rng_offset = rng_seed, rng_offset
    return c


_lib = None

# name -> (restype, argtypes); every symbol include/mme_b200.h declares
P = C.POINTER
SYMBOLS = {
    "mmeb200_create": (C.c_int, [P(C.c_void_p), C.c_int, C.c_int, C.c_uint, C.c_uint32, P(C.c_uint32), C.c_uint32]),
    "mmeb200_destroy": (None, [C.c_void_p]),
    "mmeb200_set_option": (C.c_int, [C.c_void_p, C.c_char_p, C.c_int]),
    "mmeb200_set_stream": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mmeb200_limit_num_of_threads": (C.c_int, [C.c_void_p, C.c_uint]),
    "mmeb200_bgemm": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), P(Tensor), C.c_int, P(CastParams)]),
    "mmeb200_conv": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), P(Tensor), P(Tensor), P(ConvParams), C.c_int,
                               C.c_int, P(CastParams)]),
    "mmeb200_activation": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), P(CastParams)]),
    "mmeb200_memory_write": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), C.c_int, C.c_int, C.c_int]),
    "mmeb200_convert": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), P(CastParams)]),
    "mmeb200_dma": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), C.c_int]),
    "mmeb200_get_lfsr": (C.c_int, [C.c_void_p, P(C.c_uint32), C.c_uint32, P(C.c_uint32)]),
    "mmeb200_set_lfsr": (C.c_int, [C.c_void_p, P(C.c_uint32), C.c_uint32, C.c_uint32]),
    "mmeb200_sync": (C.c_int, [C.c_void_p, C.c_uint64]),
    "mmeb200_last_error": (C.c_char_p, [C.c_void_p]),
    "mmeb200_device_count": (C.c_int, []),
    "mmeb200_malloc": (C.c_int, [C.c_void_p, P(C.c_void_p), C.c_size_t]),
    "mmeb200_free": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mmeb200_memcpy_h2d": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "mmeb200_memcpy_d2h": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t]),
    "mmeb200_memset": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_size_t]),
    "mmeb200_mem_info": (C.c_int, [C.c_void_p, P(C.c_size_t), P(C.c_size_t)]),
    "mmeb200_host_alloc": (C.c_int, [P(C.c_void_p), C.c_size_t]),
    "mmeb200_host_free": (C.c_int, [C.c_void_p]),
    "mmeb200_timer_start": (C.c_int, [C.c_void_p]),
    "mmeb200_timer_stop": (C.c_int, [C.c_void_p, P(C.c_float)]),
    "mmeb200_launch_count": (C.c_uint64, [C.c_void_p]),
    "mmeb200_version": (C.c_char_p, []),
    "mmeb200_compare": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), C.c_uint, C.c_uint, C.c_int, P(CompareResult)]),
    "mmeb200_set_accumulation": (C.c_int, [C.c_void_p, C.c_int]),
    "mmeb200_generate": (C.c_int, [C.c_void_p, P(Tensor), P(GenerateParams)]),
    "mmeb200_peer_exchange_bytes": (C.c_size_t, [C.c_uint64, C.c_int]),
    "mmeb200_peer_alloc": (C.c_int, [C.c_void_p, C.c_size_t, P(C.c_void_p), C.c_char_p]),
    "mmeb200_peer_open": (C.c_int, [C.c_void_p, C.c_char_p, P(C.c_void_p)]),
    "mmeb200_peer_close": (C.c_int, [C.c_void_p, C.c_void_p]),
    "mmeb200_conv_dedw_allreduce": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), P(Tensor), P(Tensor), P(ConvParams), P(PeerGroup)]),
    "mmeb200_gemm_splitk_static": (C.c_int, [C.c_void_p, P(Tensor), P(Tensor), P(Tensor), C.c_int, C.c_int]),
}


def load_library(path=None):
    """Load libmme_b200.so and bind every declared symbol. Raises if the library is absent."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    p = path or LIB_PATH
    if not os.path.exists(p):
        raise RuntimeError(
            "libmme_b200.so is not built (%s): run `python -c 'import __graft_entry__ as g; g.build()'` or "
            "`make -C intel_gaudi3_software_b200/csrc`. There is no CPU fallback." % p)
    lib = C.CDLL(p)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)
        fn.restype, fn.argtypes = res, args
    if path is None:
        _lib = lib
    return lib
