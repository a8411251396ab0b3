"""The torch-free harness over the C ABI (tests/native/abi_check.cu): a plain CUDA-runtime program
that calls the library the way a native consumer would and checks it against the C oracle."""
import os
import subprocess

import pytest

pytestmark = pytest.mark.gpu


def _binary():
    from mhc.cu_b200 import build
    build.build_checkers()
    assert os.path.exists(build.NATIVE_BIN), "tests/native/abi_check was not built"
    return build.NATIVE_BIN


def test_native_abi_check_passes():
    r = subprocess.run([_binary()], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "PASSED" in r.stdout


def test_native_bench_runs():
    r = subprocess.run([_binary(), "--bench"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "us per step" in r.stdout
