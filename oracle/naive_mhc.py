"""Naive (eager PyTorch, CPU) restatement of the mHC layer.  Test infrastructure only.

Each function names the reference lines it restates (paths are relative to the
AndreSlavescu/mHC.cu project).  Everything works in whatever floating dtype the
inputs carry, so the same code serves as the fp32 oracle and as the fp64 arbiter.

Shapes: ``x`` is ``[B, n, C]`` (B tokens, n residual streams, C hidden).
"""
from __future__ import annotations

import torch


def sinkhorn_knopp(E: torch.Tensor, iters: int, eps: float) -> torch.Tensor:
    """Alternating row / column normalisation of a batch of positive matrices.

    Restates the loop at src/python/tests/test_layer.py:38-41 and
    src/python/benchmarks/bench_layer.py:112-117: each step divides by ``(sum + eps)``,
    rows first, then columns.  ``E`` is ``[..., rows, cols]``.
    """
    M = E
    for _ in range(iters):
        M = M / (M.sum(dim=-1, keepdim=True) + eps)
        M = M / (M.sum(dim=-2, keepdim=True) + eps)
    return M


def rmsnorm(a: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``a / sqrt(mean(a^2) + eps) * weight`` over the last axis
    (src/python/benchmarks/bench_layer.py:119-121)."""
    rms = torch.sqrt(torch.mean(a * a, dim=-1, keepdim=True) + eps)
    return a / rms * weight


def _mix(x, H_pre, H_post, M, weight, eps):
    """Aggregate, normalise, distribute and mix, with per-token coefficients
    (src/python/tests/test_layer.py:43-50)."""
    a = torch.einsum("bi,bic->bc", H_pre, x)
    y_norm = rmsnorm(a, weight.view(1, -1), eps)
    return torch.einsum("bij,bjc->bic", M, x) + H_post.unsqueeze(-1) * y_norm.unsqueeze(1)


def dynamic_coefficients(x, phi_pre, phi_post, phi_res, alpha_pre, alpha_post, alpha_res,
                         b_pre, b_post, b_res, iters, eps):
    """Per-token H_pre, H_post and the Sinkhorn-projected mixing matrix M
    (src/python/tests/test_layer.py:22-41).  ``phi_*`` use the layer's layout
    ``[n, nC]`` / ``[n*n, nC]`` (src/python/mhc/layer.py:44-46)."""
    B, n, C = x.shape
    x_flat = x.reshape(B, n * C)
    r = torch.sqrt(torch.mean(x_flat * x_flat, dim=-1, keepdim=True) + eps)
    x_hat = x_flat / r
    t_pre = alpha_pre * (x_hat @ phi_pre.t()) + b_pre
    t_post = alpha_post * (x_hat @ phi_post.t()) + b_post
    t_res = alpha_res * (x_hat @ phi_res.t()) + b_res.reshape(1, n * n)
    H_pre = torch.sigmoid(t_pre)
    H_post = 2.0 * torch.sigmoid(t_post)
    M = sinkhorn_knopp(torch.exp(t_res).view(B, n, n), iters, eps)
    return H_pre, H_post, M


def mhc_dynamic(x, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post,
                alpha_res, b_pre, b_post, b_res, sinkhorn_iters=20, eps=1e-5):
    """Dynamic-H mHC layer, argument order of ``_naive_mhc_dynamic``
    (src/python/tests/test_layer.py:7-50)."""
    H_pre, H_post, M = dynamic_coefficients(
        x, phi_pre, phi_post, phi_res, alpha_pre, alpha_post, alpha_res,
        b_pre, b_post, b_res, sinkhorn_iters, eps)
    return _mix(x, H_pre, H_post, M, rmsnorm_weight, eps)


def mhc_dynamic_pre(x, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post,
                    alpha_res, b_pre, b_post, b_res, sinkhorn_iters=20, eps=1e-5):
    """First half of the dynamic layer, for a sub-layer F applied between the halves: the
    coefficients and the normalised aggregate ``y_hat = RMSNorm(sum_i H_pre[i] x[i,:]) * w``
    ([B, C]).  Returns ``(y_hat, H_post, M)``.  The reference's layer is monolithic
    (src/python/mhc/layer.py:61-101) with nothing between the two halves; with F = identity,
    :func:`mhc_post` of this function's outputs is exactly :func:`mhc_dynamic`."""
    H_pre, H_post, M = dynamic_coefficients(
        x, phi_pre, phi_post, phi_res, alpha_pre, alpha_post, alpha_res,
        b_pre, b_post, b_res, sinkhorn_iters, eps)
    a = torch.einsum("bi,bic->bc", H_pre, x)
    return rmsnorm(a, rmsnorm_weight.view(1, -1), eps), H_post, M


def mhc_post(x, f, H_post, M):
    """Second half: ``y[i,:] = sum_j M[i,j] x[j,:] + H_post[i] f`` with ``f = F(y_hat)`` ([B, C])
    (the distribute + mix step of src/python/tests/test_layer.py:48-50 with F's output in place
    of the normalised aggregate)."""
    return torch.einsum("bij,bjc->bic", M, x) + H_post.unsqueeze(-1) * f.unsqueeze(1)


def mhc_static(x, rmsnorm_weight, H_pre, H_post, H_res, sinkhorn_iters=20, eps=1e-5):
    """Static-H mHC layer: one sigmoid / 2*sigmoid / Sinkhorn(exp(.)) set of
    coefficients shared by all tokens (src/python/benchmarks/bench_layer.py:48-71)."""
    B, n, _ = x.shape
    hp = torch.sigmoid(H_pre).view(1, n).expand(B, n)
    hq = (2.0 * torch.sigmoid(H_post)).view(1, n).expand(B, n)
    M = sinkhorn_knopp(torch.exp(H_res), sinkhorn_iters, eps).view(1, n, n).expand(B, n, n)
    return _mix(x, hp, hq, M, rmsnorm_weight, eps)


DYNAMIC_PARAM_NAMES = ("rmsnorm_weight", "phi_pre", "phi_post", "phi_res", "alpha_pre",
                       "alpha_post", "alpha_res", "b_pre", "b_post", "b_res")
STATIC_PARAM_NAMES = ("rmsnorm_weight", "H_pre", "H_post", "H_res")


def _fwd_bwd(fn, names, x, params, dy, iters, eps, dtype):
    leaves = [x.detach().to(dtype).clone().requires_grad_(True)]
    leaves += [params[k].detach().to(dtype).clone().requires_grad_(True) for k in names]
    y = fn(*leaves, iters, eps)
    grads = torch.autograd.grad(y, leaves, grad_outputs=dy.detach().to(dtype))
    out = {"y": y.detach(), "dx": grads[0]}
    for k, g in zip(names, grads[1:]):
        out["d" + k] = g
    return out


def dynamic_fwd_bwd(x, params, dy, iters=20, eps=1e-5, dtype=torch.float32):
    """Forward + autograd backward of :func:`mhc_dynamic`; returns ``y``, ``dx`` and
    ``d<param>`` for every entry of ``DYNAMIC_PARAM_NAMES``, all in ``dtype``."""
    return _fwd_bwd(mhc_dynamic, DYNAMIC_PARAM_NAMES, x, params, dy, iters, eps, dtype)


def static_fwd_bwd(x, params, dy, iters=20, eps=1e-5, dtype=torch.float32):
    """Forward + autograd backward of :func:`mhc_static`."""
    return _fwd_bwd(mhc_static, STATIC_PARAM_NAMES, x, params, dy, iters, eps, dtype)
