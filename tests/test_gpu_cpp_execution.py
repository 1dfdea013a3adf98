"""The C++ `Execution` class over stock libtorch (include/cswap_execution.hpp),
exercised by a small driver written like the reference's drivers
(tests/cpp/execution_driver.cpp)."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_cpp_driver_lossless_policies_keep_gradients():
    from cswap_b200 import build
    exe = build.build_cpp_driver()
    r = subprocess.run([exe], capture_output=True, text=True, timeout=300)
    print(r.stdout, r.stderr[-2000:])
    assert r.returncode == 0 and "PASS" in r.stdout
    assert "policy 2:" in r.stdout and "policy 3:" in r.stdout and "policy 6:" in r.stdout
