"""Runs tests/configs/calculator_cases.json (written in the reference's JSON test-config format) on the backend and
replays every test on the CPU oracle with the calculator call sequence of MmeTestManager::runReference
(mme/mme_verification/common/mme_test_manager.cpp:766-905). The two outputs are judged by the reference's own
comparator rule, on the device (mmeb200_compare) with the test's common-dimension size; DMA tests must match bit for bit."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest

from intel_gaudi3_software_b200 import abi
from intel_gaudi3_software_b200 import config_runner as cr
from intel_gaudi3_software_b200.abi import make_tensor as T
import util

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))
CASES = os.path.join(HERE, "configs", "calculator_cases.json")
SEED = 3


def oracle_flow(oracle, t, tt, lfsr, poly):
    """runReference with the oracle as the calculator; same host tensors as the backend run."""
    return cr.run_flow(util.OracleAsCalculator(oracle, lfsr, poly), t, tt)


def dma_expected(t, tt):
    x = tt.host["x"].reshape(t["xSizes"][::-1])
    if t["operation"] == abi.OP_MEMCPY:
        return x.reshape(-1)
    return np.ascontiguousarray(np.swapaxes(x, -1, -2)).reshape(-1)


def test_config_cases_match_the_oracle(calc, best_oracle):
    tests = cr.Parser(SEED).parse_file(CASES)
    assert len(tests) == 88
    lfsr, poly = calc.get_lfsr(256)
    failures = []
    for i, t in enumerate(tests):
        if t["operation"] in (abi.OP_TRANS, abi.OP_GEMM_TRANSPOSE):
            t = dict(t, ySizes=[t["xSizes"][1], t["xSizes"][0]] + t["xSizes"][2:])
        calc.set_lfsr(lfsr, poly)
        got, tt = cr.run_test(calc, t)
        if t["operation"] in cr.DMA_OPS:
            want = dma_expected(t, tt)
            if not (got.view(np.uint8) == want.view(np.uint8)).all():
                failures.append((i, t["testName"], "dma bytes differ"))
            continue
        want = oracle_flow(best_oracle, t, tt, lfsr, poly)
        dtype, bias, mode = tt.attr[tt.out_role]
        sizes = t[tt.out_role + "Sizes"]
        bad, first = calc.compare(T(got, dtype, sizes, fp_bias=bias, inf_nan_mode=mode), T(want, dtype, sizes, fp_bias=bias, inf_nan_mode=mode),
                                  cr.common_dim_size(t))
        if bad:
            failures.append((i, t["testName"], cr.OP_NAMES[t["operation"]], cr.DTYPE_NAMES[dtype], bad, first,
                             got.reshape(-1)[first].item(), want.reshape(-1)[first].item()))
    assert not failures, failures[:10]


def test_config_cases_are_bit_identical_in_exact_mode(best_oracle):
    """With the bit-exact accumulation mode every case on bf16 / fp8 operands must reproduce the oracle's output bytes:
    accumulation, masked second GEMM, cast (stochastic rounding included) and the reduction into memory."""
    import intel_gaudi3_software_b200 as pkg
    calc = pkg.Calculator(device=0)
    calc.set_accumulation(abi.ACC_CHIP_EXACT)
    tests = cr.Parser(SEED).parse_file(CASES)
    lfsr, poly = calc.get_lfsr(256)
    checked, failures = 0, []
    narrow = (abi.BF16, abi.FP8_143, abi.FP8_152)
    have_wide = type(best_oracle).__name__ == "Ref"   # only the compiled reference models fp32 / tf32 operands
    for i, t in enumerate(tests):
        if t["operation"] in cr.DMA_OPS:
            continue
        wide = t["inTypeFloat"] in (abi.FP32, abi.TF32) and t["in2TypeFloat"] == t["inTypeFloat"]
        if wide and not have_wide:
            continue
        if not wide and (t["inTypeFloat"] not in narrow or t["in2TypeFloat"] not in narrow or
                         (t["inTypeFloat"] == abi.BF16) != (t["in2TypeFloat"] == abi.BF16)):
            continue
        calc.set_lfsr(lfsr, poly)
        got, tt = cr.run_test(calc, t)
        want = oracle_flow(best_oracle, t, tt, lfsr, poly)
        checked += 1
        if not (got.view(np.uint8) == want.view(np.uint8)).all():
            failures.append((i, t["testName"], cr.OP_NAMES[t["operation"]], int((got != want).sum())))
    calc.close()
    assert checked >= 70 and not failures, (checked, failures[:10])


def test_command_line(tmp_path):
    env = dict(os.environ, PYTHONPATH=os.path.dirname(HERE))
    p = subprocess.run([sys.executable, "-m", "intel_gaudi3_software_b200.config_runner", CASES, "--seed", str(SEED), "--dump", str(tmp_path)],
                       capture_output=True, text=True, timeout=600, env=env, cwd=os.path.dirname(HERE))
    lines = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 88, p.stdout[-2000:] + p.stderr[-2000:]
    # the transposes of this file keep ySizes = xSizes, which the calculator rejects like the reference's assert does
    errors = [l for l in lines if l["status"] != "ok"]
    assert all(l["operation"] in ("transpose", "gemm_transpose") for l in errors), errors[:3]
    assert p.returncode == (1 if errors else 0)
    assert len(os.listdir(tmp_path)) == 88 - len(errors)
    # same seed, same bytes
    p2 = subprocess.run([sys.executable, "-m", "intel_gaudi3_software_b200.config_runner", CASES, "--seed", str(SEED)],
                        capture_output=True, text=True, timeout=600, env=env, cwd=os.path.dirname(HERE))
    again = [json.loads(l) for l in p2.stdout.splitlines() if l.startswith("{")]
    assert [l.get("crc32") for l in lines] == [l.get("crc32") for l in again]
