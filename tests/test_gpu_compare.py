"""GPU parity of the device tensor comparator with TensorComparator of the compiled reference
(mme/mme_reference/tensor_comparator_impl.cpp): same verdict per element, same first mismatch, and the
partial-sum form used for dedw with several reduction splits."""
import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200.abi import make_tensor as T
from test_numerics_host import comparator_pairs

pytestmark = pytest.mark.gpu

FORMATS = ((abi.FP32, 0, 0), (abi.BF16, 0, 0), (abi.FP8_143, 7, 2), (abi.FP8_143, 3, 0), (abi.FP8_152, 15, 0), (abi.FP8_152, 24, 2))


@pytest.mark.parametrize("dtype,bias,mode", FORMATS)
def test_verdicts_match_reference(calc, ref, dtype, bias, mode):
    rng = np.random.default_rng(5)
    for cd in (1, 576, 200704):
        a, b = comparator_pairs(dtype, rng, 50000)
        equal = ref.compare_elements(dtype, bias, mode, cd, a, b)
        bad = np.nonzero(equal == 0)[0]
        got, first = calc.compare(T(a, dtype, [a.size], fp_bias=bias, inf_nan_mode=mode), T(b, dtype, [b.size], fp_bias=bias, inf_nan_mode=mode), cd)
        assert got == bad.size and bad.size > 0
        assert first == bad[0]
        # the whole-tensor verdict of the reference agrees too
        assert ref.compare(T(a, dtype, [a.size], fp_bias=bias, inf_nan_mode=mode), T(b, dtype, [b.size], fp_bias=bias, inf_nan_mode=mode), cd) is False
        a2 = a.copy()
        a2[bad] = b[bad]
        left = int((ref.compare_elements(dtype, bias, mode, cd, a2, b) == 0).sum())   # NaN / Inf never compare equal
        a2[ref.compare_elements(dtype, bias, mode, cd, a2, b) == 0] = 0
        b2 = b.copy()
        b2[ref.compare_elements(dtype, bias, mode, cd, a2, b2) == 0] = 0
        assert calc.compare(T(a2, dtype, [a.size], fp_bias=bias, inf_nan_mode=mode), T(b2, dtype, [b.size], fp_bias=bias, inf_nan_mode=mode), cd)[0] == 0
        assert ref.compare(T(a2, dtype, [a.size], fp_bias=bias, inf_nan_mode=mode), T(b2, dtype, [b.size], fp_bias=bias, inf_nan_mode=mode), cd) is True
        assert left < bad.size


@pytest.mark.parametrize("dtype,bias,mode", FORMATS + ((abi.FP8_143, 7, 1), (abi.FP8_152, 15, 1), (abi.FP8_152, 15, 2), (abi.FP8_143, 11, 0)))
def test_identical_tensors_differ_only_at_nan(calc, ref, dtype, bias, mode):
    """A tensor against its own copy: sixteen identical bytes skip the arithmetic unless one of them is a NaN, which never
    compares equal -- every bit pattern of every format, NaN codes of each Inf/NaN convention included."""
    rng = np.random.default_rng(8)
    n = 1 << 16
    size = np.dtype(abi.NP_DTYPE[dtype]).itemsize
    a = rng.integers(0, 2 ** (8 * size), n, dtype=np.uint64).astype({1: np.uint8, 2: np.uint16, 4: np.uint32}[size])   # raw bit patterns
    equal = ref.compare_elements(dtype, bias, mode, 64, a, a.copy())
    bad = np.nonzero(equal == 0)[0]
    got, first = calc.compare(T(a, dtype, [n], fp_bias=bias, inf_nan_mode=mode), T(a.copy(), dtype, [n], fp_bias=bias, inf_nan_mode=mode), 64)
    assert got == bad.size
    assert first == (bad[0] if bad.size else 2**64 - 1)
    if mode != 1:
        assert bad.size > 0


@pytest.mark.parametrize("dtype", (abi.FP32, abi.BF16))
def test_partial_sums(calc, ref, dtype):
    rng = np.random.default_rng(6)
    n, parts = 4096, 4
    full = rng.normal(0, 4, n).astype(np.float32)
    pieces = rng.normal(0, 1, (parts, n)).astype(np.float32)
    pieces[-1] = full - pieces[:-1].sum(axis=0, dtype=np.float32)
    if dtype == abi.BF16:
        to_bf16 = lambda x: ((x.view(np.uint32) + 0x7FFF + ((x.view(np.uint32) >> 16) & 1)) >> 16).astype(np.uint16)
        pa, pb = to_bf16(pieces.reshape(-1)), to_bf16(full)
    else:
        pa, pb = pieces.reshape(-1).view(np.uint32).copy(), full.view(np.uint32).copy()
    for spoil in (False, True):
        if spoil:
            pb = pb.copy()
            pb[1234] ^= np.array(1 << (pb.dtype.itemsize * 8 - 3), pb.dtype)   # an exponent bit: far outside any allowance
        ta, tb = T(pa, dtype, [n, parts]), T(pb, dtype, [n])
        want = ref.compare(ta, tb, 256, parts)
        got, first = calc.compare(ta, tb, 256, num_partials=parts)
        assert (got == 0) == want
        if spoil:
            assert got >= 1 and first <= 1234


def test_bit_exact_and_errors(calc):
    a = np.arange(1000, dtype=np.uint16)
    b = a.copy()
    assert calc.compare(T(a, abi.BF16, [1000]), T(b, abi.BF16, [1000]), 1, bit_exact=True) == (0, 2**64 - 1)
    b[[17, 400]] += 1   # one ulp: equal under the ULP rule, different bit-exactly
    assert calc.compare(T(a, abi.BF16, [1000]), T(b, abi.BF16, [1000]), 64)[0] == 0
    assert calc.compare(T(a, abi.BF16, [1000]), T(b, abi.BF16, [1000]), 64, bit_exact=True) == (2, 17)
    with pytest.raises(Exception, match="Element type"):
        calc.compare(T(a, abi.BF16, [1000]), T(a.astype(np.uint32), abi.FP32, [1000]), 1)
    with pytest.raises(Exception, match="sizes do not match"):
        calc.compare(T(a, abi.BF16, [1000]), T(b[:10].copy(), abi.BF16, [10]), 1)


def _sum_1_to_45(calc, dtype):
    """1 + 2 + ... + 45 accumulated in the tensor's own arithmetic (round to nearest even), as the reference's tests do with
    bfloat16::add / float addition (mme/tests/unit_tests/mme_unit_test.cpp:238-290): 45 read-modify-write adds on the GPU."""
    acc = np.zeros(1, abi.NP_DTYPE[dtype])
    for count in range(1, 46):
        term = np.zeros(1, abi.NP_DTYPE[dtype])
        calc.generate(T(term, dtype, [1]), abi.GEN_FILL, float(count), float(count))
        calc.do_memory_write(T(acc, dtype, [1]), T(term, dtype, [1]), abi.RED_ADD, 0)
    return acc[0]


@pytest.mark.parametrize("dtype", [abi.FP32, abi.BF16])
def test_fill_and_compare_cases_of_the_reference(calc, dtype):
    """fill_and_compare_float / _bfloat16 and comparison_failure_bf16 of the reference's unit tests (:238-392), on the device:
    a tensor filled with 1035 equals one holding 1 + ... + 45 accumulated in the tensor's type; adding 100 from element 1000
    on is reported, with the first differing element at offset 1000."""
    sizes = [64, 32, 32, 64]
    n = int(np.prod(sizes))
    filled = np.zeros(n, abi.NP_DTYPE[dtype])
    calc.generate(T(filled, dtype, sizes), abi.GEN_FILL, 1035.0, 1035.0)
    total = _sum_1_to_45(calc, dtype)
    accumulated = np.full(n, total, abi.NP_DTYPE[dtype])
    if dtype == abi.FP32:
        assert total == 1035.0
    assert calc.compare(T(filled, dtype, sizes), T(accumulated, dtype, sizes), 0)[0] == 0
    bumped = np.array([total], abi.NP_DTYPE[dtype])
    hundred = np.zeros(1, abi.NP_DTYPE[dtype])
    calc.generate(T(hundred, dtype, [1]), abi.GEN_FILL, 100.0, 100.0)
    calc.do_memory_write(T(bumped, dtype, [1]), T(hundred, dtype, [1]), abi.RED_ADD, 0)
    accumulated[1000:] = bumped[0]
    bad, first = calc.compare(T(filled, dtype, sizes), T(accumulated, dtype, sizes), 0)
    assert bad == n - 1000 and first == 1000
    assert first % sizes[0] + (first // sizes[0] % sizes[1]) * sizes[0] == 1000   # the reference's own check of the offset
