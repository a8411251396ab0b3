"""Pins the CPU oracle to the reference: the oracle must reproduce the golden vectors
that tests/golden/make_golden.py drew from the reference's own naive implementation
(src/python/tests/test_layer.py:7-50, src/python/benchmarks/bench_layer.py:27-145)."""
import os

import pytest
import torch

import oracle
from helpers import DYN_PARAMS, STATIC_PARAMS, assert_rel, golden_names, load_golden


@pytest.mark.parametrize("name", golden_names("dyn"))
def test_dynamic_oracle_matches_golden_fp64(name):
    g = load_golden(name)
    params = {k: g[k] for k in DYN_PARAMS}
    out = oracle.dynamic_fwd_bwd(g["x"], params, g["dy"], g["iters"], g["eps"], dtype=torch.float64)
    assert_rel(out["y"], g["y"], 1e-12, "y")
    assert_rel(out["dx"], g["dx"], 1e-11, "dx")
    for k in DYN_PARAMS:
        assert_rel(out["d" + k], g["d" + k], 1e-10, "d" + k)


@pytest.mark.parametrize("name", golden_names("dyn"))
def test_dynamic_oracle_fp32_within_1e5(name):
    """The fp32 oracle itself sits well inside the 1e-5 parity band around the fp64 truth."""
    g = load_golden(name)
    params = {k: g[k] for k in DYN_PARAMS}
    out = oracle.dynamic_fwd_bwd(g["x"], params, g["dy"], g["iters"], g["eps"], dtype=torch.float32)
    assert_rel(out["y"], g["y"], 1e-5, "y")
    assert_rel(out["dx"], g["dx"], 1e-5, "dx")


@pytest.mark.parametrize("name", golden_names("static"))
def test_static_oracle_matches_golden_fp64(name):
    g = load_golden(name)
    params = {k: g[k] for k in STATIC_PARAMS}
    out = oracle.static_fwd_bwd(g["x"], params, g["dy"], g["iters"], g["eps"], dtype=torch.float64)
    assert_rel(out["y"], g["y"], 1e-12, "y")
    assert_rel(out["dx"], g["dx"], 1e-11, "dx")
    for k in STATIC_PARAMS:
        assert_rel(out["d" + k], g["d" + k], 1e-10, "d" + k)


@pytest.mark.parametrize("name", golden_names("sinkhorn"))
def test_sinkhorn_oracle_matches_golden(name):
    g = load_golden(name)
    out = oracle.sinkhorn_knopp(g["inp"], g["iters"], g["eps"])
    assert_rel(out, g["out"], 1e-12, "sinkhorn out")
    d = oracle.sinkhorn_backward(g["grad_out"], g["inp"], g["iters"], g["eps"])
    assert_rel(d, g["grad_inp"], 1e-9, "sinkhorn grad")


def test_sinkhorn_doubly_stochastic():
    """32x32, 20 iterations, eps 1e-8: rows and columns sum to one within 1e-5
    (the property src/python/tests/test_ops.py:7-18 asserts)."""
    g = load_golden("sinkhorn_32x32_t20")
    out = oracle.sinkhorn_knopp(g["inp"].float(), g["iters"], g["eps"])
    assert (out >= 0).all()
    assert float((out.sum(-1) - 1).abs().max()) < 1e-5
    assert float((out.sum(-2) - 1).abs().max()) < 1e-5


_REFERENCE = os.environ.get("MHC_REFERENCE_CHECKOUT", os.path.join(os.sep, "root", "reference"))


@pytest.mark.skipif(not os.path.isdir(os.path.join(_REFERENCE, "src", "python")),
                    reason="reference checkout not present (set MHC_REFERENCE_CHECKOUT)")
def test_oracle_matches_live_reference():
    """When a checkout of the reference is present, also compare live on fresh inputs."""
    import importlib.util

    spec = importlib.util.spec_from_file_location(
        "ref_test_layer", os.path.join(_REFERENCE, "src", "python", "tests", "test_layer.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    gen = torch.Generator().manual_seed(123)
    B, n, C = 7, 4, 40
    r = lambda *s, sc=1.0: torch.randn(*s, generator=gen, dtype=torch.float64) * sc
    args = [r(B, n, C), r(C, sc=0.3) + 1, r(n, n * C, sc=0.02), r(n, n * C, sc=0.02), r(n * n, n * C, sc=0.02),
            torch.tensor(0.4).double(), torch.tensor(0.5).double(), torch.tensor(0.6).double(),
            r(n, sc=0.3), r(n, sc=0.3), r(n, n, sc=0.3)]
    ref = mod._naive_mhc_dynamic(*args, 20, 1e-5)
    ours = oracle.mhc_dynamic(*args, 20, 1e-5)
    assert_rel(ours, ref, 1e-13, "y live")


# ---- the C restatement used by the torch-free native harness ------------------------------------
def _c_oracle():
    import ctypes

    from mhc.cu_b200 import build
    build.build_checkers()
    lib = ctypes.CDLL(build.ORACLE_LIB)
    lib.naive_mhc_dynamic_forward.restype = ctypes.c_int
    return lib


@pytest.mark.parametrize("name", golden_names("dyn"))
def test_c_oracle_forward_matches_golden(name):
    """oracle/naive_mhc.c (plain C, fp64) against the vectors drawn from the reference's naive layer."""
    import ctypes

    import numpy as np
    g = load_golden(name)
    x = np.ascontiguousarray(g["x"].double().numpy())
    B, n, C = x.shape
    phi = np.ascontiguousarray(np.concatenate(
        [g[k].double().numpy() for k in ("phi_pre", "phi_post", "phi_res")], 0))
    alpha = np.array([float(g["alpha_pre"]), float(g["alpha_post"]), float(g["alpha_res"])])
    bias = np.concatenate([g[k].double().numpy().ravel() for k in ("b_pre", "b_post", "b_res")])
    w = np.ascontiguousarray(g["rmsnorm_weight"].double().numpy())
    y = np.empty_like(x)
    ptr = lambda a: a.ctypes.data_as(ctypes.c_void_p)   # noqa: E731
    rc = _c_oracle().naive_mhc_dynamic_forward(
        ptr(x), ptr(w), ptr(phi), ptr(alpha), ptr(bias), ctypes.c_long(B), int(n), ctypes.c_long(C),
        int(g["iters"]), ctypes.c_double(float(g["eps"])), ptr(y))
    assert rc == 0
    ref = g["y"].double().numpy()
    assert np.abs(y - ref).max() / np.abs(ref).max() < 1e-12
