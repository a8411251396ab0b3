"""The drop-in Python API on the GPU: the reference's own test list
(src/python/tests/test_layer.py, test_ops.py of AndreSlavescu/mHC.cu) restated against ``mhc``,
with value checks where the reference only checks shapes."""
import pytest
import torch

import oracle
from helpers import assert_rel

pytestmark = pytest.mark.gpu


def _layer(C, n, dynamic, **kw):
    from mhc import MHCLayer
    torch.manual_seed(42)
    return MHCLayer(hidden_dim=C, expansion_rate=n, use_dynamic_h=dynamic, **kw).cuda()


@pytest.mark.parametrize("dynamic", [False, True])
def test_forward_backward_finite(dynamic):
    B, n, C = 8, 4, 128
    layer = _layer(C, n, dynamic)
    x = (torch.randn(B, n, C, device="cuda") + 0.1).requires_grad_(True)
    out = layer(x)
    assert out.shape == (B, n, C) and out.dtype == torch.float32
    out.sum().backward()
    assert torch.isfinite(out).all() and torch.isfinite(x.grad).all()
    for name, p in layer.named_parameters():
        assert p.grad is not None, name
        assert p.grad.shape == p.shape and p.grad.dtype == p.dtype, name
        assert torch.isfinite(p.grad.float()).all(), name


def test_dynamic_params_get_nonzero_grads():
    """Every dynamic parameter receives gradient (src/python/tests/test_layer.py:118-142 of the
    reference).  A random dy is used: under loss = y.sum() the gradient reaching phi_res / b_res /
    alpha_res is zero up to rounding, because dM is then constant along each column and the
    column normalisation of Sinkhorn projects that out (the fp64 naive layer gives ~1e-22)."""
    layer = _layer(64, 4, True)
    x = (torch.randn(4, 4, 64, device="cuda") + 0.1).requires_grad_(True)
    y = layer(x)
    y.backward(torch.randn_like(y))
    for name in ["phi_pre", "phi_post", "phi_res", "b_pre", "b_post", "b_res", "alpha_pre",
                 "alpha_post", "alpha_res"]:
        assert getattr(layer, name).grad.abs().sum() > 0, name


def test_dynamic_matches_naive_small():
    """B=2, n=4, C=16, 3 iterations as in test_layer.py:145-193, but at 1e-5 on every gradient."""
    layer = _layer(16, 4, True, sinkhorn_iters=3)
    x = torch.randn(2, 4, 16, device="cuda", requires_grad=True)
    out = layer(x)
    out.sum().backward()
    params = {k: v.detach().cpu() for k, v in layer.named_parameters()}
    ref = oracle.dynamic_fwd_bwd(x.detach().cpu(), params, torch.ones(2, 4, 16), 3, layer.eps,
                                 dtype=torch.float64)
    assert_rel(out, ref["y"], 1e-5, "y")
    assert_rel(x.grad, ref["dx"], 1e-5, "dx")
    for k, p in layer.named_parameters():
        tol = 1e-2 if p.dtype == torch.bfloat16 else 1e-5      # bf16 parameter -> bf16 gradient
        assert_rel(p.grad, ref["d" + k], tol, "d" + k)


def test_static_matches_naive():
    layer = _layer(128, 4, False)
    with torch.no_grad():
        layer.H_pre.normal_()
        layer.H_post.normal_()
        layer.H_res.normal_()
    x = torch.randn(8, 4, 128, device="cuda", requires_grad=True)
    dy = torch.randn(8, 4, 128, device="cuda")
    out = layer(x)
    out.backward(dy)
    params = {k: v.detach().cpu() for k, v in layer.named_parameters()}
    ref = oracle.static_fwd_bwd(x.detach().cpu(), params, dy.cpu(), layer.sinkhorn_iters, layer.eps,
                                dtype=torch.float64)
    assert_rel(out, ref["y"], 1e-5, "y")
    assert_rel(x.grad, ref["dx"], 1e-5, "dx")
    for k in ("H_pre", "H_post", "H_res"):
        assert_rel(getattr(layer, k).grad, ref["d" + k], 1e-5, k)
    layer.eval()
    with torch.no_grad():
        assert_rel(layer(x), ref["y"], 1e-5, "inference y")


def test_parameter_names_and_shapes():
    C, n = 128, 4
    p = dict(_layer(C, n, False).named_parameters())
    assert set(p) == {"rmsnorm_weight", "H_pre", "H_post", "H_res"}
    assert p["rmsnorm_weight"].shape == (C,) and p["rmsnorm_weight"].dtype == torch.bfloat16
    assert p["H_pre"].shape == (n,) and p["H_post"].shape == (n,) and p["H_res"].shape == (n, n)
    p = dict(_layer(C, n, True).named_parameters())
    assert set(p) == {"rmsnorm_weight", "phi_pre", "phi_post", "phi_res", "b_pre", "b_post", "b_res",
                      "alpha_pre", "alpha_post", "alpha_res"}
    assert p["phi_pre"].shape == (n, n * C) and p["phi_res"].shape == (n * n, n * C)
    assert p["b_res"].shape == (n, n) and p["alpha_res"].shape == ()


@pytest.mark.parametrize("dynamic", [False, True])
def test_training_steps_and_batch_sizes(dynamic):
    layer = _layer(128, 4, dynamic)
    opt = torch.optim.Adam(layer.parameters(), lr=1e-3)
    x = torch.randn(8, 4, 128, device="cuda")
    target = torch.randn(8, 4, 128, device="cuda")
    losses = []
    for _ in range(3):
        opt.zero_grad()
        loss = ((layer(x) - target) ** 2).mean()
        loss.backward()
        opt.step()
        losses.append(float(loss.detach()))
    assert all(l == l for l in losses) and losses[-1] < losses[0]
    for B in (1, 4, 16, 32):
        assert layer(torch.randn(B, 4, 128, device="cuda")).shape == (B, 4, 128)


def test_phi_cache_follows_parameter_updates():
    """The packed bf16/fp32 copy of phi is rebuilt when the parameters change in place."""
    layer = _layer(64, 4, True)
    x = torch.randn(4, 4, 64, device="cuda")
    with torch.no_grad():
        layer.alpha_res.fill_(0.5)
        y0 = layer(x).clone()
        layer.phi_res.mul_(3.0)
        y1 = layer(x)
    assert not torch.allclose(y0, y1)
    params = {k: v.detach().cpu() for k, v in layer.named_parameters()}
    ref = oracle.mhc_dynamic(x.cpu().double(), *[params[k].double() for k in oracle.naive_mhc.DYNAMIC_PARAM_NAMES],
                             layer.sinkhorn_iters, layer.eps)
    assert_rel(y1, ref, 1e-5, "y after update")


@pytest.mark.parametrize("dynamic", [False, True])
def test_deterministic_and_stable(dynamic):
    layer = _layer(128, 4, dynamic)
    x = torch.randn(8, 4, 128, device="cuda")
    assert torch.equal(layer(x), layer(x))
    for s in (100.0, 1e-3):
        assert torch.isfinite(layer(x * s)).all()


def test_bf16_streams_stay_bf16():
    layer = _layer(256, 4, True)
    x = torch.randn(16, 4, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    y = layer(x)
    assert y.dtype == torch.bfloat16
    y.float().sum().backward()
    assert x.grad.dtype == torch.bfloat16 and layer.phi_res.grad.dtype == torch.float32


def test_state_dict_round_trip():
    a, b = _layer(64, 4, True), _layer(64, 4, True)
    with torch.no_grad():
        for p in a.parameters():
            p.add_(torch.randn_like(p.float()).to(p.dtype) * 0.1)
    b.load_state_dict(a.state_dict())
    x = torch.randn(4, 4, 64, device="cuda")
    assert torch.equal(a(x), b(x))


@pytest.mark.parametrize("n", [8, 32])
def test_other_expansion_rates_through_the_layer(n):
    """n = 8 and n = 32 as in the reference's benchmark table (README.md:86-104 of the reference)."""
    layer = _layer(64, n, True)
    x = torch.randn(6, n, 64, device="cuda", requires_grad=True)
    dy = torch.randn(6, n, 64, device="cuda")
    y = layer(x)
    y.backward(dy)
    params = {k: v.detach().cpu() for k, v in layer.named_parameters()}
    ref = oracle.dynamic_fwd_bwd(x.detach().cpu(), params, dy.cpu(), layer.sinkhorn_iters, layer.eps,
                                 dtype=torch.float64)
    assert_rel(y, ref["y"], 1e-5, "y")
    assert_rel(x.grad, ref["dx"], 1e-5, "dx")
    assert_rel(layer.phi_res.grad, ref["dphi_res"], 1e-5, "dphi_res")


def test_default_is_dynamic():
    from mhc import MHCLayer
    assert MHCLayer(hidden_dim=128, expansion_rate=4).use_dynamic_h is True


def test_ops_sinkhorn_and_rmsnorm_autograd():
    from mhc import rmsnorm, sinkhorn_knopp
    inp = (torch.rand(16, 16, device="cuda") + 0.1).requires_grad_(True)
    sinkhorn_knopp(inp, num_iters=10).sum().backward()
    assert torch.isfinite(inp.grad).all()
    x = (torch.randn(8, 128, device="cuda") + 0.1).requires_grad_(True)
    w = torch.ones(128, device="cuda", requires_grad=True)
    out = rmsnorm(x, w)
    assert out.dtype == torch.bfloat16 and out.shape == (8, 128)
    out.float().sum().backward()
    assert x.grad is not None and w.grad is not None
