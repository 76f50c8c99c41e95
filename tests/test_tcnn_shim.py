"""The C++ mirror of the tiny-cuda-nn objects on the path (include/neus2b_tcnn.hpp): it compiles against the C ABI, its
host-side checks pass without a GPU, and on a GPU every result equals the direct C-ABI call."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BIN = os.path.join(ROOT, "tests", "cpp", "_build", "test_tcnn_shim")


def ensure_built():
    if not os.path.exists(BIN):
        import sys
        sys.path.insert(0, ROOT)
        import __graft_entry__ as G
        from neus2_b200 import build as b
        b.build()
        G.build_cpp_tests()
    return BIN


def test_shim_compiles_and_host_checks_pass():
    r = subprocess.run([ensure_built(), "--check-only"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "host checks ok" in r.stdout


@pytest.mark.gpu
def test_shim_matches_c_abi_on_gpu():
    r = subprocess.run([ensure_built()], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "shim test ok" in r.stdout
