"""The reference's OWN test configurations on the GPU.

tests/golden/reference_corpus_cases.json holds what these files of the reference's corpus expand to (written by
tests/golden/make_corpus_cases.py where the reference checkout is present):

    gaudi3/configs/basic_tests/basic_{fwd,dedx,dedw,ab,abt,atb,atbt,ab_strides,fwd_strides,dual_gemm}.json
    gaudi3/configs/numerics/numerics_fp8.json
    gaudi2/configs/stochastic_rounding.json

Every test runs through the config runner on the B200 backend and is replayed, on the same generated tensors (strided
ones included), by the CPU oracle with the calculator call sequence of MmeTestManager::runReference
(mme/mme_verification/common/mme_test_manager.cpp:766-905). Outputs are judged by the reference's comparator rule on the
device (mmeb200_compare, the test's common-dimension size), on the logical elements of strided outputs; and where the operands
allow it the run is repeated in the bit-exact accumulation mode and must reproduce the oracle's bytes.
"""
import json
import os

import numpy as np
import pytest

import intel_gaudi3_software_b200 as pkg
from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200 import config_runner as cr
from intel_gaudi3_software_b200.abi import make_tensor as T
import util

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURE = os.path.join(HERE, "golden", "reference_corpus_cases.json")
EXPECTED_COUNTS = {"basic_fwd": 14, "basic_dedx": 12, "basic_dedw": 12, "basic_ab": 1, "basic_abt": 1, "basic_atb": 1, "basic_atbt": 1,
                   "basic_ab_strides": 1, "basic_fwd_strides": 1, "basic_dual_gemm": 14, "numerics_fp8": 216, "stochastic_rounding": 2}


def load_cases():
    with open(FIXTURE) as f:
        doc = json.load(f)
    for rel, entry in doc["files"].items():
        tests = []
        for diff in entry["tests"]:
            t = cr.default_test()
            t.update(diff)
            tests.append(t)
        yield rel, entry["chip"], tests, entry["rejected"]


def narrow_same_kind(t):
    narrow = (abi.BF16, abi.FP8_143, abi.FP8_152)
    a, b = t["inTypeFloat"], t["in2TypeFloat"]
    return a in narrow and b in narrow and (a == abi.BF16) == (b == abi.BF16)


@pytest.mark.parametrize("rel,chip,tests,rejected", list(load_cases()), ids=lambda v: os.path.basename(v) if isinstance(v, str) else None)
def test_reference_corpus_file(best_oracle, rel, chip, tests, rejected):
    if chip != abi.CHIP_GAUDI3 and type(best_oracle).__name__ != "Ref":
        pytest.skip("only the compiled reference models the Gaudi2 chip")
    calc = pkg.Calculator(chip=chip, device=0)
    exact = pkg.Calculator(chip=chip, device=0, accumulation=abi.ACC_CHIP_EXACT) if chip == abi.CHIP_GAUDI3 else None
    lfsr, poly = calc.get_lfsr(256)
    ran, ran_exact, failures = 0, 0, []
    for i, t in enumerate(tests):
        calc.set_lfsr(lfsr, poly)
        got, tt = cr.run_test(calc, t)
        want = cr.run_flow(util.OracleAsCalculator(best_oracle, lfsr.copy(), poly, chip), t, tt)
        role = tt.out_role
        dtype, bias, mode = tt.attr[role]
        g, w = tt.logical(role, got), tt.logical(role, want)
        bad, first = calc.compare(T(g, dtype, [g.size], fp_bias=bias, inf_nan_mode=mode), T(w, dtype, [w.size], fp_bias=bias, inf_nan_mode=mode),
                                  cr.common_dim_size(t))
        ran += 1
        if bad:
            failures.append((i, t["testName"], cr.OP_NAMES[t["operation"]], cr.DTYPE_NAMES[dtype], bad, first, g[first].item(), w[first].item()))
        if tt.strides(role) is not None:   # the gaps of a strided output keep what the output buffer held
            mask = np.ones(got.size, bool)
            tt._view(role, mask)[...] = False
            assert (got[mask] == tt.host[role][mask]).all(), (i, t["testName"], "gaps were written")
        if exact is not None and narrow_same_kind(t):
            exact.set_lfsr(lfsr, poly)
            got_e, _ = cr.run_test(exact, t, tt)
            ran_exact += 1
            if not (tt.logical(role, got_e).view(np.uint8) == w.view(np.uint8)).all():
                failures.append((i, t["testName"], "exact mode", int((tt.logical(role, got_e) != w).sum())))
    calc.close()
    if exact is not None:
        exact.close()
    print("%s: %d tests run (%d also bit-exact), %d skipped by name %s" % (rel, ran, ran_exact, len(rejected), [r["name"] for r in rejected]))
    assert ran == len(tests) and not failures, (rel, failures[:8])
