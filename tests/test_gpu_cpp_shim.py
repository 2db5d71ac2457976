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
