"""Runs the C++ test program of the header layer (include/anygpu) on the GPU; it checks the tensor_<op> templates against
the CPU oracle and exits non-zero on any failure."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, os.path.join(ROOT, "tests", "cpp"))


@pytest.mark.gpu
def test_cpp_header_layer(tmp_path):
    import build as cpp_build
    exe = cpp_build.OUT
    if not os.path.exists(exe):
        exe = cpp_build.build()
    r = subprocess.run([exe, str(tmp_path)], capture_output=True, text=True, timeout=300)
    sys.stdout.write(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "FAILED" not in r.stdout and "PASSED" in r.stdout
