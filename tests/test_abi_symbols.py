"""CPU-side checks of the boundary: the shared library loads without a GPU and exports every
symbol that include/mhc_b200.h declares; the ctypes table matches the header."""
import os
import re

import pytest

from mhc.cu_b200 import _lib as L
from mhc.cu_b200 import build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "mhc_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mhc_[a-z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def lib():
    build.build_lib()
    return L.lib()


def test_every_declared_symbol_is_exported(lib):
    names = _header_functions()
    assert len(names) >= 12
    for name in names:
        assert hasattr(lib, name), f"{name} declared in include/mhc_b200.h but not exported"


def test_ctypes_table_matches_header():
    assert sorted(L.SIGNATURES) == _header_functions()


def test_status_strings_and_workspace_sizes(lib):
    assert lib.mhc_abi_version() >= 1
    assert lib.mhc_status_string(0) == b"ok"
    for code in range(1, 9):
        assert lib.mhc_status_string(code) not in (b"", b"unknown status")
    # sizes grow with the problem and bad shapes are refused
    small = lib.mhc_workspace_bytes(L.OP_DYNAMIC_BWD, 16, 4, 64, 20, L.BF16)
    big = lib.mhc_workspace_bytes(L.OP_DYNAMIC_BWD, 1280, 4, 2560, 20, L.BF16)
    assert 0 < small < big < (1 << 30)
    bad = (1 << 64) - 1
    assert lib.mhc_workspace_bytes(L.OP_DYNAMIC_FWD, 16, 0, 64, 20, L.BF16) == bad
    assert lib.mhc_workspace_bytes(L.OP_DYNAMIC_FWD, 16, 33, 64, 20, L.BF16) == bad
    assert lib.mhc_workspace_bytes(L.OP_DYNAMIC_FWD, -1, 4, 64, 20, L.BF16) == bad
    assert lib.mhc_workspace_bytes(99, 16, 4, 64, 20, L.BF16) == bad


def test_validation_happens_before_any_cuda_call(lib):
    """Argument errors are reported without touching the device (works with no GPU present)."""
    assert lib.mhc_dynamic_fwd(*([None] * 13), 4, 4, 64, 20, 1e-5, 0, None, 0, None) == 1
    assert lib.mhc_sinkhorn_fwd(None, None, 1, 40, 20, 1e-6, None) == 2
    assert lib.mhc_rmsnorm_fwd(None, None, None, None, 4, 0, 1e-5, None) == 2


def test_torch_extension_exports_the_reference_binding_names():
    """mhc_cuda (the C++ torch extension) builds without a GPU and carries the nine function names
    of the reference's pybind module (src/python/bindings.cu:544-554)."""
    build.build_lib()
    build.build_ext()
    from mhc.cu_b200 import mhc_cuda
    for name in ["sinkhorn_knopp_fwd", "sinkhorn_knopp_bwd", "rmsnorm_fwd", "rmsnorm_bwd",
                 "mhc_layer_fwd", "mhc_layer_fwd_inference", "mhc_layer_bwd",
                 "mhc_layer_fwd_dynamic", "mhc_layer_bwd_dynamic"]:
        assert hasattr(mhc_cuda, name), name
    assert mhc_cuda.abi_version() == L.lib().mhc_abi_version()
    import torch
    with pytest.raises(RuntimeError):           # CPU tensors are refused, nothing falls back
        mhc_cuda.sinkhorn_knopp_fwd(torch.ones(4, 4), 3, 1e-5)
