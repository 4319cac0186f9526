"""Runs tests/cpp/reference_style.cpp: user code written against the reference's include paths and
its C++ API (class Array, op::), compiled with this back end's headers and linked with its library."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_reference_style_cpp_program():
    from dali_b200 import build
    exe = build.build_program(os.path.join(ROOT, "tests", "cpp", "reference_style.cpp"),
                              os.path.join(ROOT, "dali_b200", "lib", "reference_style_tests"))
    r = subprocess.run([exe], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-4000:] + r.stderr[-2000:]
    assert r.stdout.strip().splitlines()[-1].startswith("PASS")
