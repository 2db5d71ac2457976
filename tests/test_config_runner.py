"""The JSON test-config parser (the format of mme/mme_verification/common/config_parser.cpp) on the CPU: expansion,
defaults, value names, random sizes; and, where a checkout of the reference is present, that every calculator-level
config of its corpus parses."""
import glob
import json
import os

import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200 import config_runner as cr

HERE = os.path.dirname(os.path.abspath(__file__))
CASES = os.path.join(HERE, "configs", "calculator_cases.json")


def by_name(tests, name):
    return [t for t in tests if t["testName"] == name]


def test_cartesian_expansion_and_defaults():
    tests = cr.Parser(3).parse_file(CASES)
    assert len(tests) == 88
    fwd = by_name(tests, "fwd 3x3 pad 1")
    # last multi-valued key varies fastest; shape keys never multiply
    assert [(t["outTypeFloat"], t["reluEn"]) for t in fwd] == [(abi.BF16, False), (abi.BF16, True), (abi.FP32, False), (abi.FP32, True)]
    assert fwd[0]["xSizes"] == [48, 13, 9, 1, 3] and fwd[0]["padding"] == [1, 1, 0]
    assert fwd[0]["in2TypeFloat"] == abi.BF16 and fwd[0]["conversionRoundingMode"] == 0 and fwd[0]["reductionOp"] == abi.RED_NONE
    assert set(fwd[0]["ignored"]) == {"geometry", "convPattern"}
    assert [t["seed"] for t in tests] == list(range(3, 3 + 88))           # seed + index, as in the reference
    assert not by_name(tests, "skipped")


def test_random_sizes_are_consistent():
    tests = cr.Parser(11).parse_file(CASES)
    t3d, = by_name(tests, "fwd 3d stride 2 dilation 2")
    assert t3d["xSizes"] == [20, 11, 7, 5, 2]
    for t in by_name(tests, "bgemm orientations"):
        x, w, y = t["xSizes"], t["wSizes"], t["ySizes"]
        ta, tb = t["operation"] in (abi.OP_ATB, abi.OP_ATBT), t["operation"] in (abi.OP_ABT, abi.OP_ATBT)
        cd_x, m = (x[1], x[0]) if ta else (x[0], x[1])
        cd_w, n = (w[0], w[1]) if tb else (w[1], w[0])
        assert cd_x == cd_w and y[:2] == [n, m] and x[2:] == w[2:] == y[2:]
        assert cr.common_dim_size(t) == cd_x


def test_fp8_attributes():
    tests = by_name(cr.Parser(5).parse_file(CASES), "fp8 numerics")
    assert len(tests) == 48
    for t in tests:
        assert t["in2TypeFloat"] in (t["inTypeFloat"], abi.FP8_143)
        a = cr.tensor_attributes(t)
        assert a["out"] == "y" and a["x"][2] == abi.INFNAN_MINIMAL
        for role, key in (("x", "inTypeFloat"), ("w", "in2TypeFloat"), ("y", "outTypeFloat")):
            dtype, bias, _ = a[role]
            assert dtype == t[key]
            if dtype == abi.FP8_143:
                assert bias in (3, 7, 11, 15)
            elif dtype == abi.FP8_152:
                assert 1 <= bias <= 30
            else:
                assert bias == 0
    assert {t["conversionRoundingMode"] for t in tests} == {0, 1, 4}


def test_roles_follow_the_operation():
    p = cr.Parser(1)
    base = [{"inTypeFloat": ["fp8_143"]}, {"in2TypeFloat": ["bf16"]}, {"outTypeFloat": ["fp32"]}, {"fp8BiasIn": ["11"]}]
    dedx, = p.parse({"tests": [base + [{"operation": ["dedx"]}]]})
    assert cr.tensor_attributes(dedx) == {"y": (abi.FP8_143, 11, 0), "w": (abi.BF16, 0, 0), "x": (abi.FP32, 0, 0), "out": "x"}
    dedw, = p.parse({"tests": [base + [{"operation": ["dedw"]}]]})
    assert cr.tensor_attributes(dedw)["out"] == "w" and cr.tensor_attributes(dedw)["y"][0] == abi.BF16


def test_errors():
    p = cr.Parser(1)
    with pytest.raises(cr.ConfigError):
        cr.Parser(0)
    with pytest.raises(cr.ConfigError, match="fp16"):
        p.parse({"tests": [[{"inTypeFloat": ["fp16"]}, {"operation": ["ab"]}]]})
    with pytest.raises(cr.ConfigError, match="operation"):
        p.parse({"tests": [[{"inTypeFloat": ["bf16"]}, {"operation": ["maskedFlashAttention"]}]]})
    with pytest.raises(cr.ConfigError, match="invalid value"):
        p.parse({"tests": [[{"inTypeFloat": ["bf16"]}, {"operation": ["ab"]}, {"conversionRoundingMode": ["nearest"]}]]})
    with pytest.raises(cr.ConfigError):
        p.parse({"nothing": []})


from oracle.oracle import reference_root  # noqa: E402

REF_CONFIGS = os.path.join(reference_root() or "", "mme", "mme_verification")


@pytest.mark.skipif(reference_root() is None, reason="no checkout of the reference here")
def test_reference_corpus_parses():
    """Every config of the reference's corpus is read; tests on fp16 operands are counted as rejected,
    everything else must parse into runnable test descriptions."""
    files = sorted(glob.glob(os.path.join(REF_CONFIGS, "*", "configs", "**", "*.json"), recursive=True))
    assert len(files) > 20
    parsed = rejected = 0
    for path in files:
        doc = cr.load_config(path)
        for test in doc.get("tests", []):
            try:
                parsed += len(cr.Parser(7).parse({"tests": [test]}))
            except cr.ConfigError:
                rejected += 1
    assert parsed > 500 and parsed > 3 * rejected, (parsed, rejected)


def test_corpus_fixture_lists_the_named_files():
    """tests/golden/reference_corpus_cases.json (the GPU corpus test's input) holds the expansion of these files of the reference."""
    import json
    with open(os.path.join(os.path.dirname(__file__), "golden", "reference_corpus_cases.json")) as f:
        doc = json.load(f)
    names = {os.path.splitext(os.path.basename(rel))[0]: len(e["tests"]) for rel, e in doc["files"].items()}
    assert names == {"basic_fwd": 14, "basic_dedx": 12, "basic_dedw": 12, "basic_ab": 1, "basic_abt": 1, "basic_atb": 1, "basic_atbt": 1,
                     "basic_ab_strides": 1, "basic_fwd_strides": 1, "basic_dual_gemm": 14, "numerics_fp8": 216, "stochastic_rounding": 2}


def test_dual_gemm_becomes_two_tests_and_strided_tensors_keep_their_gaps():
    doc = {"tests": [[{"testName": ["dual"]}, {"inTypeFloat": ["bf16"]}, {"outTypeFloat": ["fp32"]}, {"operation": ["ab"]}, {"dualGemm": ["true"]},
                      {"xSizes": ["12", "7"]}, {"wSizes": ["5", "12"]}, {"ySizes": ["5", "7"]},
                      {"xSizes2": ["9", "4"]}, {"wSizes2": ["3", "9"]}, {"ySizes2": ["3", "4"]},
                      {"xStrides": ["1", "16", "200", "200", "200"]}]]}
    first, second = cr.Parser(3).parse(doc)
    assert first["xSizes"][:2] == [12, 7] and second["xSizes"][:2] == [9, 4] and second["ySizes"][:2] == [3, 4]
    assert not first["dualGemm"] and not second["dualGemm"] and first["seed"] != second["seed"]

    class FillOnes:   # stands in for the device generator: every generated value is 1.0 (bf16 0x3F80)
        def generate(self, tensor, kind, lo=0.0, hi=0.0, mean=0.0, std=0.0, seed=0, packing=0, level=0):
            n = int(np.prod(list(tensor.sizes)))
            np.frombuffer((cr.abi.C.c_uint16 * n).from_address(tensor.data), dtype=np.uint16)[:] = 0x3F80
    tt = cr.TestTensors(first, FillOnes())
    assert tt.strides("x") == [1, 16, 200, 200, 200] and tt.span("x") == 1 + 11 + 6 * 16 and tt.strides("w") is None
    buf = tt.host["x"]
    assert buf.size == tt.span("x") and (tt.logical("x", buf) == 0x3F80).all() and int((buf == 0x3F80).sum()) == 12 * 7
    desc = tt.tensor("x")
    assert list(desc.strides)[:2] == [1, 16] and list(desc.sizes)[:2] == [12, 7]
