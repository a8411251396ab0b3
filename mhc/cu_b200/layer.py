"""``MHCLayer``: same constructor, parameter names, shapes, dtypes and initialisation as the
reference module (src/python/mhc/layer.py:6-101 of AndreSlavescu/mHC.cu), so its state_dict loads
unchanged."""
from __future__ import annotations

import torch
import torch.nn as nn

from .ops import (mhc_layer_fused, mhc_layer_fused_dynamic, mhc_layer_fused_inference, mhc_post,
                  mhc_pre)


class MHCLayer(nn.Module):
    """Manifold-constrained hyper-connection layer over ``[B, n, C]`` residual streams.

    Args:
        hidden_dim: C.
        expansion_rate: n, the number of residual streams (1..32; tuned kernels for n <= 8).
        sinkhorn_iters: Sinkhorn-Knopp iterations.
        eps: the one epsilon shared by both RMS norms and by Sinkhorn.
        alpha_init: initial value of the three alpha scalars (and scale of the static H_res).
        use_dynamic_h: per-token H computed from x (True) or one learned H shared by all tokens.
    """

    def __init__(self, hidden_dim: int, expansion_rate: int = 4, sinkhorn_iters: int = 20,
                 eps: float = 1e-5, alpha_init: float = 0.01, use_dynamic_h: bool = True):
        super().__init__()
        self.hidden_dim = hidden_dim
        self.expansion_rate = expansion_rate
        self.sinkhorn_iters = sinkhorn_iters
        self.eps = eps
        self.use_dynamic_h = use_dynamic_h
        n, C = expansion_rate, hidden_dim
        nC = n * C
        self.rmsnorm_weight = nn.Parameter(torch.ones(C, dtype=torch.bfloat16))
        if use_dynamic_h:
            self.phi_pre = nn.Parameter(torch.randn(n, nC) * 0.02)
            self.phi_post = nn.Parameter(torch.randn(n, nC) * 0.02)
            self.phi_res = nn.Parameter(torch.randn(n * n, nC) * 0.02)
            self.b_pre = nn.Parameter(torch.zeros(n))
            self.b_post = nn.Parameter(torch.zeros(n))
            self.b_res = nn.Parameter(torch.zeros(n, n))
            self.alpha_pre = nn.Parameter(torch.tensor(alpha_init))
            self.alpha_post = nn.Parameter(torch.tensor(alpha_init))
            self.alpha_res = nn.Parameter(torch.tensor(alpha_init))
        else:
            self.H_pre = nn.Parameter(torch.zeros(n, dtype=torch.float32))
            self.H_post = nn.Parameter(torch.zeros(n, dtype=torch.float32))
            self.H_res = nn.Parameter((alpha_init * torch.randn(n, n)).float())

    def forward(self, x_expanded: torch.Tensor) -> torch.Tensor:
        B, n, C = x_expanded.shape
        assert n == self.expansion_rate
        assert C == self.hidden_dim
        if self.use_dynamic_h:
            return mhc_layer_fused_dynamic(
                x_expanded, self.rmsnorm_weight, self.phi_pre, self.phi_post, self.phi_res,
                self.alpha_pre, self.alpha_post, self.alpha_res, self.b_pre, self.b_post,
                self.b_res, self.sinkhorn_iters, self.eps)
        if not self.training and not torch.is_grad_enabled():
            return mhc_layer_fused_inference(x_expanded, self.rmsnorm_weight, self.H_pre,
                                             self.H_post, self.H_res, self.sinkhorn_iters, self.eps)
        return mhc_layer_fused(x_expanded, self.rmsnorm_weight, self.H_pre, self.H_post, self.H_res,
                               self.sinkhorn_iters, self.eps)


class MHCBlock(nn.Module):
    """A dynamic-H :class:`MHCLayer` wrapped around a sub-layer ``fn`` (attention, MLP, ...):

        y_hat, H_post, M = pre(x)          aggregate the n streams, RMSNorm      [B, C]
        f = fn(y_hat)                      the caller's module, any autograd     [B, C]
        y = M x + H_post f                 distribute + mix                      [B, n, C]

    The reference layer has no such hook (src/python/mhc/layer.py:61-101 computes distribute + mix
    directly on the normalised aggregate); with ``fn = nn.Identity()`` this block computes exactly
    what ``layer(x)`` computes.  The parameters are the wrapped layer's."""

    def __init__(self, layer: MHCLayer, fn: nn.Module):
        super().__init__()
        if not layer.use_dynamic_h:
            raise ValueError("MHCBlock needs a dynamic-H MHCLayer")
        if layer.expansion_rate > 8:
            raise ValueError("the split kernels cover expansion rates up to 8")
        self.layer, self.fn = layer, fn

    def forward(self, x_expanded: torch.Tensor) -> torch.Tensor:
        L = self.layer
        y_hat, H_post, M = mhc_pre(
            x_expanded, L.rmsnorm_weight, L.phi_pre, L.phi_post, L.phi_res, L.alpha_pre,
            L.alpha_post, L.alpha_res, L.b_pre, L.b_post, L.b_res, L.sinkhorn_iters, L.eps)
        f = self.fn(y_hat)
        return mhc_post(x_expanded, f, H_post, M)
