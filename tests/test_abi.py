"""The C-ABI shared library: it loads, exports every symbol include/mme_b200.h declares, its structs
have the declared layout, and without a GPU it refuses to run instead of computing on the CPU."""
import ctypes as C
import os
import re

import pytest

from intel_gaudi3_software_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "mme_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mmeb200_[a-z0-9_]+)\s*\(", text)))


def test_header_and_binding_agree():
    assert declared_symbols() == sorted(abi.SYMBOLS)


def test_library_exports_every_declared_symbol():
    lib = abi.load_library()
    for name in declared_symbols():
        assert hasattr(lib, name), name
    assert lib.mmeb200_version().startswith(b"mme_b200")


def test_struct_layouts():
    assert C.sizeof(abi.Tensor) == 72 and abi.Tensor.data.offset == 64
    assert C.sizeof(abi.ConvParams) == 60
    assert C.sizeof(abi.CastParams) == 48 and abi.CastParams.rng_seed.offset == 32


def test_null_arguments_are_rejected():
    lib = abi.load_library()
    assert lib.mmeb200_create(None, 2, 0, 0, 0, None, 0) == abi.ERR_INVALID_ARG
    assert lib.mmeb200_sync(None, 0) == abi.ERR_INVALID_ARG
    assert lib.mmeb200_bgemm(None, None, None, None, abi.OP_AB, None) == abi.ERR_INVALID_ARG
    assert lib.mmeb200_last_error(None) == b"null context"


def test_no_cpu_fallback_without_a_gpu():
    lib = abi.load_library()
    if lib.mmeb200_device_count() > 0:
        pytest.skip("a GPU is visible")
    ctx = C.c_void_p()
    assert lib.mmeb200_create(C.byref(ctx), abi.CHIP_GAUDI3, 0, 0, 0, None, 0) == abi.ERR_NO_DEVICE
    assert not ctx.value
    import intel_gaudi3_software_b200 as pkg
    with pytest.raises(pkg.MmeError):
        pkg.Calculator()


def test_missing_library_fails_loudly(tmp_path):
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        abi.load_library(str(tmp_path / "nope.so"))
