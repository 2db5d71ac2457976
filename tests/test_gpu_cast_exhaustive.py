"""Every one of the 2^32 fp32 bit patterns through the casts that the GEMM epilogue and doActivation use for the
deterministic rounding modes, on the GPU, proven equal to the CPU oracle without casting 2^32 values on the CPU:

  * the GPU casts consecutive bit patterns in chunks; the host finds every place where the output code changes;
  * the oracle is evaluated on both neighbours of every change point and on the ends of every chunk (a few hundred thousand
    values per cast instead of 2^32).

A deterministic rounding of fp32 into a narrower format is monotone in the bit pattern within a sign (NaNs map to one code),
so the oracle is constant wherever it agrees at both ends of a run of constant GPU output: agreement at all change points is
agreement everywhere. The cases take the hardware-conversion tiers (cvt.rn.bf16x2, cvt.rn.satfinite.e4m3x2 / e5m2x2 with
the fix-ups for the other Inf/NaN conventions and biases) and the straight-line tiers (toward zero, up, down)."""
import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T

pytestmark = pytest.mark.gpu

CHUNK = 1 << 28
CASES = [
    # out dtype, bias, Inf/NaN mode, rounding, clip
    (abi.BF16, 0, 0, abi.RM_NE, False),          # hardware bf16 conversion
    (abi.BF16, 0, 0, abi.RM_DOWN, True),         # straight-line bf16 cast, directed, clipped
    (abi.FP8_143, 7, 2, abi.RM_NE, True),        # hardware e4m3 conversion, its own convention
    (abi.FP8_143, 11, 0, abi.RM_NE, False),      # hardware conversion + rescale + the 'full' convention's Inf / NaN codes
    (abi.FP8_152, 20, 2, abi.RM_Z, False),       # straight-line fp8 cast, toward zero, 'minimal' convention on 1-5-2
]


def oracle_cast(port, bits, od, bias, mode, rm, clip):
    if od == abi.BF16:
        return port.fp32_to_bf16(bits, rm, None, clip)
    return port.fp32_to_fp8(bits, 4 if od == abi.FP8_143 else 5, bias, rm, None, False, clip, False, False, mode)


@pytest.mark.parametrize("od,bias,mode,rm,clip", CASES)
def test_all_fp32_inputs(calc, port, od, bias, mode, rm, clip):
    cp = abi.make_cast_params(rm, clip_fp=clip)
    out_t = abi.NP_DTYPE[od]
    d_in, d_out = calc.alloc(CHUNK * 4), calc.alloc(CHUNK * abi.ELEM_SIZE[od])
    dev = abi.MEM_DEVICE
    checked = 0
    bits = np.arange(0, CHUNK, dtype=np.uint32)
    for lo in range(0, 1 << 32, CHUNK):
        if lo:
            bits += np.uint32(CHUNK)
        d_in.upload(bits)
        calc.do_activation(T(d_out.ptr, od, [CHUNK], fp_bias=bias, inf_nan_mode=mode, mem_space=dev), T(d_in.ptr, abi.FP32, [CHUNK], mem_space=dev), cp)
        got = d_out.download(out_t)
        change = np.flatnonzero(got[1:] != got[:-1])
        idx = np.unique(np.concatenate([[0, CHUNK - 1], change, change + 1]))
        want = oracle_cast(port, bits[idx], od, bias, mode, rm, clip)
        bad = np.flatnonzero(want != got[idx])
        assert bad.size == 0, (hex(int(bits[idx[bad[0]]])), hex(int(got[idx[bad[0]]])), hex(int(want[bad[0]])), int(bad.size))
        # within a sign and away from NaNs the GPU's output must be monotone in the bit pattern, as the argument above needs
        finite = (bits & 0x7FFFFFFF) <= 0x7F800000
        if finite.all():
            width = 16 if od == abi.BF16 else 8
            mag = (got & ((1 << (width - 1)) - 1)).astype(np.int32)
            assert (np.diff(mag) >= 0).all(), "output magnitude is not monotone in the input magnitude"
        checked += idx.size
    assert checked > 200
    d_in.free()
    d_out.free()
