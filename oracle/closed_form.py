"""Closed-form backward of the mHC layer, phase by phase.  Test infrastructure only.

``naive_mhc`` gets its gradients from autograd; this file writes the same gradients
out by hand, in the order the CUDA kernels compute them (row reductions over one
token, small per-token algebra incl. the Sinkhorn backward, then the element-wise
``dx`` pass and the token-summed parameter gradients).  ``tests/test_closed_form.py``
checks it against autograd of the naive layer in fp64, which is what makes it a
trustworthy statement of the kernels' algorithm.

The Sinkhorn backward differentiates every normalisation step exactly:
for ``y = x / (s + eps)`` with ``s = sum_axis(x)``,
``dx = (dy - sum_axis(dy * y)) / (s + eps)``.  (The reference kernel at
src/csrc/kernels/sinkhorn_knopp.cuh:650-685 drops the ``1/(s+eps)`` factors; the
parity target is autograd of the naive layer, so they are kept here.)
"""
from __future__ import annotations

import torch


def sinkhorn_forward_denominators(E, iters, eps):
    """Forward Sinkhorn that also returns the ``(s + eps)`` vectors of all 2*iters
    steps: ``row_den[t]`` is ``[..., n, 1]``, ``col_den[t]`` is ``[..., 1, n]``."""
    M = E
    row_den, col_den = [], []
    for _ in range(iters):
        d = M.sum(dim=-1, keepdim=True) + eps
        M = M / d
        row_den.append(d)
        d = M.sum(dim=-2, keepdim=True) + eps
        M = M / d
        col_den.append(d)
    return M, row_den, col_den


def sinkhorn_backward(dM, E, iters, eps):
    """Gradient of ``sinkhorn_knopp(E)`` w.r.t. ``E`` given ``dM``.

    Walks the 2*iters steps in reverse.  The input of a step is rebuilt from its
    output as ``x = y * (s + eps)``, so only the denominators are kept from the
    forward sweep (this is what the CUDA kernel does as well)."""
    y, row_den, col_den = sinkhorn_forward_denominators(E, iters, eps)
    d = dM
    for t in reversed(range(iters)):
        cd = col_den[t]
        d = (d - (d * y).sum(dim=-2, keepdim=True)) / cd
        y = y * cd
        rd = row_den[t]
        d = (d - (d * y).sum(dim=-1, keepdim=True)) / rd
        y = y * rd
    return d


def _mix_backward(x, g, w, H_pre, H_post, M, eps):
    """Everything the backward needs from one token's rows of ``x`` and ``g``:
    gradients w.r.t. the coefficients and the coefficient-independent part of dx."""
    B, n, C = x.shape
    a = torch.einsum("bi,bic->bc", H_pre, x)
    rho = torch.sqrt((a * a).mean(dim=-1, keepdim=True) + eps)
    y_norm = a / rho * w.view(1, C)
    dyh = torch.einsum("bi,bic->bc", H_post, g)
    dH_post = torch.einsum("bic,bc->bi", g, y_norm)
    dM = torch.einsum("bic,bjc->bij", g, x)
    dw = (dyh * a / rho).sum(dim=0)
    u = dyh * w.view(1, C)
    s = (u * a).sum(dim=-1, keepdim=True)
    da = u / rho - a * s / (C * rho ** 3)
    dH_pre = torch.einsum("bc,bic->bi", da, x)
    dx = torch.einsum("bij,bic->bjc", M, g) + H_pre.unsqueeze(-1) * da.unsqueeze(1)
    return dx, dw, dH_pre, dH_post, dM


def dynamic_backward_closed_form(x, params, dy, iters=20, eps=1e-5, dtype=torch.float64):
    """Hand-written fwd+bwd of the dynamic-H layer.  Same return keys as
    ``naive_mhc.dynamic_fwd_bwd``."""
    p_ = {k: v.detach().to(dtype) for k, v in params.items()}
    x = x.detach().to(dtype)
    g = dy.detach().to(dtype)
    B, n, C = x.shape
    nC = n * C
    w = p_["rmsnorm_weight"]
    phi = torch.cat([p_["phi_pre"], p_["phi_post"], p_["phi_res"].reshape(n * n, nC)], dim=0)
    alpha = torch.cat([p_["alpha_pre"].reshape(1).expand(n), p_["alpha_post"].reshape(1).expand(n),
                       p_["alpha_res"].reshape(1).expand(n * n)])
    bias = torch.cat([p_["b_pre"].reshape(n), p_["b_post"].reshape(n), p_["b_res"].reshape(n * n)])

    x_flat = x.reshape(B, nC)
    r = torch.sqrt((x_flat * x_flat).mean(dim=-1, keepdim=True) + eps)
    p = (x_flat @ phi.t()) / r                      # normalised projections [B, K]
    t = alpha * p + bias
    H_pre = torch.sigmoid(t[:, :n])
    H_post = 2.0 * torch.sigmoid(t[:, n:2 * n])
    E = torch.exp(t[:, 2 * n:]).view(B, n, n)
    M, _, _ = sinkhorn_forward_denominators(E, iters, eps)

    a = torch.einsum("bi,bic->bc", H_pre, x)
    rho = torch.sqrt((a * a).mean(dim=-1, keepdim=True) + eps)
    y = torch.einsum("bij,bjc->bic", M, x) + H_post.unsqueeze(-1) * (a / rho * w).unsqueeze(1)

    dx, dw, dH_pre, dH_post, dM = _mix_backward(x, g, w, H_pre, H_post, M, eps)
    dE = sinkhorn_backward(dM, E, iters, eps)
    dt = torch.cat([dH_pre * H_pre * (1.0 - H_pre),
                    dH_post * H_post * (1.0 - H_post / 2.0),
                    (dE * E).reshape(B, n * n)], dim=1)          # [B, K]
    db = dt.sum(dim=0)
    dtp = dt * p
    dalpha = torch.stack([dtp[:, :n].sum(), dtp[:, n:2 * n].sum(), dtp[:, 2 * n:].sum()])
    # sum of |terms| behind each alpha gradient: the scale against which its rounding error is
    # meaningful (the signed sum itself can cancel to almost nothing)
    dalpha_scale = torch.stack([dtp[:, :n].abs().sum(), dtp[:, n:2 * n].abs().sum(),
                                dtp[:, 2 * n:].abs().sum()])
    dpr = dt * alpha / r                             # dp / r
    dphi = dpr.t() @ x_flat
    qq = (dpr * p).sum(dim=-1, keepdim=True) / (nC * r)
    dx = dx + (dpr @ phi - x_flat * qq).view(B, n, C)

    return {
        "y": y, "dx": dx, "drmsnorm_weight": dw,
        "dphi_pre": dphi[:n], "dphi_post": dphi[n:2 * n], "dphi_res": dphi[2 * n:],
        "dalpha_pre": dalpha[0], "dalpha_post": dalpha[1], "dalpha_res": dalpha[2],
        "db_pre": db[:n], "db_post": db[n:2 * n], "db_res": db[2 * n:].view(n, n),
        "scale_dalpha_pre": dalpha_scale[0], "scale_dalpha_post": dalpha_scale[1],
        "scale_dalpha_res": dalpha_scale[2],
    }


def static_backward_closed_form(x, params, dy, iters=20, eps=1e-5, dtype=torch.float64):
    """Hand-written fwd+bwd of the static-H layer.  Same return keys as
    ``naive_mhc.static_fwd_bwd``."""
    p_ = {k: v.detach().to(dtype) for k, v in params.items()}
    x = x.detach().to(dtype)
    g = dy.detach().to(dtype)
    B, n, C = x.shape
    w = p_["rmsnorm_weight"]
    hp = torch.sigmoid(p_["H_pre"])
    hq = 2.0 * torch.sigmoid(p_["H_post"])
    E = torch.exp(p_["H_res"])
    M, _, _ = sinkhorn_forward_denominators(E, iters, eps)
    H_pre = hp.view(1, n).expand(B, n)
    H_post = hq.view(1, n).expand(B, n)
    Mb = M.view(1, n, n).expand(B, n, n)

    a = torch.einsum("bi,bic->bc", H_pre, x)
    rho = torch.sqrt((a * a).mean(dim=-1, keepdim=True) + eps)
    y = torch.einsum("bij,bjc->bic", Mb, x) + H_post.unsqueeze(-1) * (a / rho * w).unsqueeze(1)

    dx, dw, dH_pre, dH_post, dM = _mix_backward(x, g, w, H_pre, H_post, Mb, eps)
    dE = sinkhorn_backward(dM.sum(dim=0), E, iters, eps)
    return {
        "y": y, "dx": dx, "drmsnorm_weight": dw,
        "dH_pre": dH_pre.sum(dim=0) * hp * (1.0 - hp),
        "dH_post": dH_post.sum(dim=0) * hq * (1.0 - hq / 2.0),
        "dH_res": dE * E,
    }
