"""Runs the C++ caller of the atb:: API (tests/cpp/atb_cpp_api_test.cpp), built against the same
headers and shared library a C++ application would use."""
import os
import subprocess

import pytest

from helpers import pkg


def _exe():
    return pkg._build.build_cpp_test()


def test_cpp_contract_checks():
    r = subprocess.run([_exe(), "cpu"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "cpu checks passed" in r.stdout


@pytest.mark.gpu
def test_cpp_decode_step_on_gpu():
    r = subprocess.run([_exe(), "gpu"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "gpu checks passed" in r.stdout
