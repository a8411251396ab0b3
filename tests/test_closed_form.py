"""The hand-derived backward (oracle/closed_form.py — the algorithm the CUDA kernels
follow) against autograd of the naive layer, in fp64 and on the golden vectors."""
import pytest
import torch

import oracle
from helpers import DYN_PARAMS, STATIC_PARAMS, assert_rel, golden_names, load_golden


@pytest.mark.parametrize("name", golden_names("dyn"))
def test_dynamic_closed_form(name):
    g = load_golden(name)
    params = {k: g[k] for k in DYN_PARAMS}
    out = oracle.dynamic_backward_closed_form(g["x"], params, g["dy"], g["iters"], g["eps"])
    assert_rel(out["y"], g["y"], 1e-12, "y")
    assert_rel(out["dx"], g["dx"], 1e-10, "dx")
    for k in DYN_PARAMS:
        assert_rel(out["d" + k], g["d" + k], 1e-9, "d" + k)


@pytest.mark.parametrize("name", golden_names("static"))
def test_static_closed_form(name):
    g = load_golden(name)
    params = {k: g[k] for k in STATIC_PARAMS}
    out = oracle.static_backward_closed_form(g["x"], params, g["dy"], g["iters"], g["eps"])
    assert_rel(out["y"], g["y"], 1e-12, "y")
    assert_rel(out["dx"], g["dx"], 1e-10, "dx")
    for k in STATIC_PARAMS:
        assert_rel(out["d" + k], g["d" + k], 1e-9, "d" + k)


def test_sinkhorn_backward_fp32_reconstruction_error():
    """Rebuilding each step's input as y*(s+eps) in fp32 keeps the gradient within 1e-5
    of the fp64 value on well-conditioned inputs (what the bf16 path relies on)."""
    gen = torch.Generator().manual_seed(0)
    E = torch.exp(torch.randn(64, 4, 4, generator=gen, dtype=torch.float64) * 0.5)
    dM = torch.randn(64, 4, 4, generator=gen, dtype=torch.float64)
    d64 = oracle.sinkhorn_backward(dM, E, 20, 1e-6)
    d32 = oracle.sinkhorn_backward(dM.float(), E.float(), 20, 1e-6)
    assert_rel(d32, d64, 2e-5, "fp32 sinkhorn backward")


def test_sinkhorn_backward_rectangular_matches_autograd():
    """The closed-form Sinkhorn backward on a single rectangular matrix (rows != columns)."""
    torch.manual_seed(3)
    E = torch.exp(torch.randn(12, 7, dtype=torch.float64) * 0.5).requires_grad_(True)
    dM = torch.randn(12, 7, dtype=torch.float64)
    out = oracle.sinkhorn_knopp(E, 9, 1e-6)
    (out * dM).sum().backward()
    d = oracle.sinkhorn_backward(dM, E.detach(), 9, 1e-6)
    assert float((d - E.grad).abs().max() / E.grad.abs().max()) < 1e-10
