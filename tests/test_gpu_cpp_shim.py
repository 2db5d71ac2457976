"""Runs the C++ drop-in (the reference's CPUCalculator API over the C ABI) through the calculator cases
of the reference's own unit tests, restated in intel_gaudi3_software_b200/cpp/shim_unit_tests.cpp."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "intel_gaudi3_software_b200", "cpp", "_build", "shim_unit_tests")


def test_reference_unit_test_cases_pass_on_the_drop_in():
    if not os.path.exists(BIN):
        pytest.skip("cpp/_build/shim_unit_tests is not built (needs the reference checkout at build time)")
    p = subprocess.run([BIN], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "all passed" in p.stdout


SYN_BIN = os.path.join(ROOT, "intel_gaudi3_software_b200", "cpp", "_build", "syn_wrapper_tests")


def test_synapse_facing_helpers():
    """calculate* / check* of synapse/tests/utils/cpu_calculator.h on the backend, against exact small-integer cases."""
    if not os.path.exists(SYN_BIN):
        pytest.skip("cpp/_build/syn_wrapper_tests is not built (needs the reference checkout at build time)")
    p = subprocess.run([SYN_BIN], capture_output=True, text=True, timeout=300)
    assert p.returncode == 0, p.stdout[-2000:] + p.stderr[-2000:]
    assert "all passed" in p.stdout
