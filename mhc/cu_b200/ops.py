"""autograd Functions and functional wrappers with the reference's names and argument order
(src/python/mhc/ops.py of AndreSlavescu/mHC.cu), running on the sm_100a kernels.

Differences from the reference, all deliberate:
  * bf16 ``x`` stays bf16 end to end (the reference up-casts every input to fp32 and returns fp32,
    ops.py:404 / bindings.cu:462); fp32 ``x`` gives fp32 ``y`` exactly as before, other dtypes are
    computed in fp32.
  * alpha stays on the device (no ``.item()`` synchronisation, ops.py:178-188) and the packed /
    cast copy of phi is cached per parameter version instead of being rebuilt every call
    (ops.py:172-177).
  * the backward is exact and runs entirely in kernels (no per-token Python loop, ops.py:309-316).
"""
from __future__ import annotations

import weakref

import torch
from torch.autograd import Function

_EXT = None


def _ext():
    """The C++ torch extension ``mhc_cuda`` (mhc/cu_b200/csrc/torch_ext.cpp), which allocates
    outputs and forwards to the C ABI.  There is no Python or CPU substitute."""
    global _EXT
    if _EXT is None:
        try:
            from . import mhc_cuda
        except ImportError as e:
            raise ImportError(
                "mhc_cuda extension not built: run `python -m mhc.cu_b200.build` (needs nvcc and "
                "g++); there is no fallback path") from e
        _EXT = mhc_cuda
    return _EXT


_PACK_CACHE: dict = {}
_PACK_CACHE_MAX = 16


def _key(*tensors):
    return tuple((t.data_ptr(), t._version, t.dtype, tuple(t.shape)) for t in tensors)


def pack_phi(phi_pre, phi_post, phi_res, dtype):
    """[K, nC] concatenation (pre, post, res) of the three projection matrices in ``dtype``.
    Cached on (storage, version) so an unchanged parameter set is packed once."""
    key = (_key(phi_pre, phi_post, phi_res), dtype)
    hit = _PACK_CACHE.get(key)
    if hit is not None:
        packed, refs = hit
        # an address can be handed out again once its tensor is gone: the entry only counts while
        # the tensors it was packed from are still alive
        if all(r() is t for r, t in zip(refs, (phi_pre, phi_post, phi_res))):
            return packed
        del _PACK_CACHE[key]
    nC = phi_pre.shape[-1]
    with torch.no_grad():
        packed = torch.cat([phi_pre.reshape(-1, nC), phi_post.reshape(-1, nC), phi_res.reshape(-1, nC)],
                           dim=0).to(dtype).contiguous()
    if len(_PACK_CACHE) >= _PACK_CACHE_MAX:
        _PACK_CACHE.pop(next(iter(_PACK_CACHE)))
    _PACK_CACHE[key] = (packed, tuple(weakref.ref(t) for t in (phi_pre, phi_post, phi_res)))
    return packed


def _compute_dtype(x):
    return torch.bfloat16 if x.dtype == torch.bfloat16 else torch.float32


class SinkhornKnoppFunction(Function):
    @staticmethod
    def forward(ctx, inp, num_iters, eps):
        inp = inp.contiguous()
        out = _ext().sinkhorn_knopp_fwd(inp, num_iters, eps)
        ctx.save_for_backward(inp)
        ctx.num_iters = num_iters
        ctx.eps = eps
        return out

    @staticmethod
    def backward(ctx, grad_output):
        (inp,) = ctx.saved_tensors
        d_inp = _ext().sinkhorn_knopp_bwd(grad_output.contiguous().float(), inp, ctx.num_iters,
                                          ctx.eps)
        return d_inp, None, None


class RMSNormFunction(Function):
    @staticmethod
    def forward(ctx, inp, weight, eps):
        inp = inp.contiguous()
        weight = weight.contiguous()
        out, rms = _ext().rmsnorm_fwd(inp, weight, eps)
        ctx.save_for_backward(inp, weight, rms)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        inp, weight, rms = ctx.saved_tensors
        d_inp, d_weight = _ext().rmsnorm_bwd(grad_output.contiguous().bfloat16(), inp, weight, rms)
        return d_inp, d_weight.to(weight.dtype), None


def sinkhorn_knopp(inp, num_iters=20, eps=1e-8):
    return SinkhornKnoppFunction.apply(inp.float(), num_iters, eps)


def rmsnorm(inp, weight, eps=1e-5):
    return RMSNormFunction.apply(inp.bfloat16(), weight.bfloat16(), eps)


class MHCLayerFunction(Function):
    """Static-H layer.  apply(x, rmsnorm_weight, H_pre, H_post, H_res, sinkhorn_iters, eps)."""

    @staticmethod
    def forward(ctx, x_expanded, rmsnorm_weight, H_pre, H_post, H_res, sinkhorn_iters, eps):
        x = x_expanded.contiguous()
        w = rmsnorm_weight.contiguous()
        H_res = H_res.contiguous()
        y, rms, hp, hq, M = _ext().mhc_layer_fwd(x, w, H_pre.contiguous(), H_post.contiguous(),
                                                 H_res, sinkhorn_iters, eps)
        ctx.save_for_backward(x, w, H_res, rms, hp, hq, M)
        ctx.sinkhorn_iters = sinkhorn_iters
        ctx.eps = eps
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x, w, H_res, rms, hp, hq, M = ctx.saved_tensors
        dx, d_w, d_hp, d_hq, d_hr = _ext().mhc_layer_bwd(
            grad_output.contiguous().to(x.dtype), x, w, H_res, rms, hp, hq, M, ctx.sinkhorn_iters,
            ctx.eps)
        return dx, d_w.to(w.dtype), d_hp, d_hq, d_hr, None, None


def mhc_layer_fused(x_expanded, rmsnorm_weight, H_pre, H_post, H_res, sinkhorn_iters=20, eps=1e-5):
    return MHCLayerFunction.apply(
        x_expanded.to(_compute_dtype(x_expanded)), rmsnorm_weight.bfloat16(), H_pre.float(),
        H_post.float(), H_res.float(), sinkhorn_iters, eps)


def mhc_layer_fused_inference(x_expanded, rmsnorm_weight, H_pre, H_post, H_res, sinkhorn_iters=20,
                              eps=1e-5):
    """Forward only; nothing is saved for a backward pass."""
    x = x_expanded.to(_compute_dtype(x_expanded)).contiguous()
    return _ext().mhc_layer_fwd_inference(
        x, rmsnorm_weight.bfloat16().contiguous(), H_pre.float().contiguous(),
        H_post.float().contiguous(), H_res.float().contiguous(), sinkhorn_iters, eps)


class MHCLayerDynamicFunction(Function):
    """Dynamic-H layer.  apply(x, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post,
    alpha_res, b_pre, b_post, b_res, sinkhorn_iters, eps) -> y; backward returns the 11 gradients
    and two None, in that order."""

    @staticmethod
    def forward(ctx, x_expanded, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post,
                alpha_res, b_pre, b_post, b_res, sinkhorn_iters, eps):
        x = x_expanded.contiguous()
        w = rmsnorm_weight.contiguous()
        n = phi_pre.size(0)
        phi = pack_phi(phi_pre, phi_post, phi_res, x.dtype)
        dev = x.device
        alpha = torch.stack([torch.as_tensor(a, dtype=torch.float32, device=dev).reshape(())
                             for a in (alpha_pre, alpha_post, alpha_res)]).float()
        bias = torch.cat([b_pre.reshape(-1), b_post.reshape(-1), b_res.reshape(-1)]).float()
        y, rms, rms_h, hp, hq, M, proj, den = _ext().mhc_layer_fwd_dynamic(
            x, w, phi, alpha, bias, sinkhorn_iters, eps)
        ctx.save_for_backward(x, w, phi, alpha, bias, rms, rms_h, hp, hq, M, proj, den)
        ctx.sinkhorn_iters = sinkhorn_iters
        ctx.eps = eps
        ctx.n = n
        ctx.param_dtypes = (w.dtype, phi_pre.dtype, phi_post.dtype, phi_res.dtype,
                            getattr(alpha_pre, "dtype", torch.float32),
                            getattr(alpha_post, "dtype", torch.float32),
                            getattr(alpha_res, "dtype", torch.float32),
                            b_pre.dtype, b_post.dtype, b_res.dtype)
        ctx.b_res_shape = tuple(b_res.shape)
        ctx.phi_res_shape = tuple(phi_res.shape)
        return y

    @staticmethod
    def backward(ctx, grad_output):
        x, w, phi, alpha, bias, rms, rms_h, H_pre, H_post, M, proj, den = ctx.saved_tensors
        dx, d_w, d_phi, d_alpha, d_bias = _ext().mhc_layer_bwd_dynamic(
            grad_output.contiguous().to(x.dtype), x, w, phi, alpha, bias, rms, rms_h, H_pre, H_post,
            M, proj, den, ctx.sinkhorn_iters, ctx.eps)
        n = ctx.n
        dt = ctx.param_dtypes
        return (dx, d_w.to(dt[0]),
                d_phi[:n].to(dt[1]), d_phi[n:2 * n].to(dt[2]),
                d_phi[2 * n:].reshape(ctx.phi_res_shape).to(dt[3]),
                d_alpha[0].to(dt[4]), d_alpha[1].to(dt[5]), d_alpha[2].to(dt[6]),
                d_bias[:n].to(dt[7]), d_bias[n:2 * n].to(dt[8]),
                d_bias[2 * n:].reshape(ctx.b_res_shape).to(dt[9]), None, None)


def mhc_layer_fused_dynamic(x_expanded, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre,
                            alpha_post, alpha_res, b_pre, b_post, b_res, sinkhorn_iters=20,
                            eps=1e-5):
    dev, pdt = phi_pre.device, phi_pre.dtype
    if not torch.is_tensor(alpha_pre):
        alpha_pre = torch.tensor(alpha_pre, device=dev, dtype=pdt)
    if not torch.is_tensor(alpha_post):
        alpha_post = torch.tensor(alpha_post, device=dev, dtype=pdt)
    if not torch.is_tensor(alpha_res):
        alpha_res = torch.tensor(alpha_res, device=dev, dtype=pdt)
    return MHCLayerDynamicFunction.apply(
        x_expanded.to(_compute_dtype(x_expanded)), rmsnorm_weight.bfloat16(), phi_pre.float(),
        phi_post.float(), phi_res.float(), alpha_pre, alpha_post, alpha_res, b_pre.float(),
        b_post.float(), b_res.float(), sinkhorn_iters, eps)


# ---- the dynamic layer in two halves around a caller's sub-layer F -------------------------------
class MHCPreFunction(Function):
    """First half: apply(x, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post,
    alpha_res, b_pre, b_post, b_res, sinkhorn_iters, eps) -> (y_hat [B, C], H_post [B, n],
    M [B, n, n]).  y_hat feeds the sub-layer; H_post and M go to :class:`MHCPostFunction`, whose
    backward hands their gradients back here."""

    @staticmethod
    def forward(ctx, x_expanded, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post,
                alpha_res, b_pre, b_post, b_res, sinkhorn_iters, eps):
        from . import capi
        x = x_expanded.contiguous()
        w = rmsnorm_weight.contiguous()
        n = phi_pre.size(0)
        phi = pack_phi(phi_pre, phi_post, phi_res, x.dtype)
        dev = x.device
        alpha = torch.stack([torch.as_tensor(a, dtype=torch.float32, device=dev).reshape(())
                             for a in (alpha_pre, alpha_post, alpha_res)]).float()
        bias = torch.cat([b_pre.reshape(-1), b_post.reshape(-1), b_res.reshape(-1)]).float()
        y_hat, sv = capi.dynamic_pre_fwd(x, w, phi, alpha, bias, sinkhorn_iters, eps)
        ctx.save_for_backward(x, w, phi, alpha, bias, sv["rms"], sv["rms_h"], sv["H_pre"],
                              sv["H_post"], sv["proj"])
        ctx.sinkhorn_iters, ctx.eps, ctx.n = sinkhorn_iters, eps, n
        ctx.param_dtypes = (w.dtype, phi_pre.dtype, phi_post.dtype, phi_res.dtype,
                            getattr(alpha_pre, "dtype", torch.float32),
                            getattr(alpha_post, "dtype", torch.float32),
                            getattr(alpha_res, "dtype", torch.float32),
                            b_pre.dtype, b_post.dtype, b_res.dtype)
        ctx.b_res_shape = tuple(b_res.shape)
        ctx.phi_res_shape = tuple(phi_res.shape)
        return y_hat, sv["H_post"], sv["M"]

    @staticmethod
    def backward(ctx, d_y_hat, dH_post, dM):
        from . import capi
        x, w, phi, alpha, bias, rms, rms_h, H_pre, H_post, proj = ctx.saved_tensors
        B, n = x.shape[0], ctx.n
        if d_y_hat is None:
            d_y_hat = torch.zeros(B, x.shape[2], dtype=x.dtype, device=x.device)
        if dH_post is None:
            dH_post = torch.zeros(B, n, dtype=torch.float32, device=x.device)
        if dM is None:
            dM = torch.zeros(B, n, n, dtype=torch.float32, device=x.device)
        saved = {"rms": rms, "rms_h": rms_h, "H_pre": H_pre, "H_post": H_post, "proj": proj}
        dx, g = capi.dynamic_pre_bwd(d_y_hat.contiguous().to(x.dtype), dH_post.contiguous().float(),
                                     dM.contiguous().float(), x, w, phi, alpha, bias, saved,
                                     ctx.sinkhorn_iters, ctx.eps)
        dt = ctx.param_dtypes
        d_phi, d_alpha, d_bias = g["d_phi"], g["d_alpha"], g["d_bias"]
        return (dx, g["d_rmsnorm_weight"].to(dt[0]),
                d_phi[:n].to(dt[1]), d_phi[n:2 * n].to(dt[2]),
                d_phi[2 * n:].reshape(ctx.phi_res_shape).to(dt[3]),
                d_alpha[0].to(dt[4]), d_alpha[1].to(dt[5]), d_alpha[2].to(dt[6]),
                d_bias[:n].to(dt[7]), d_bias[n:2 * n].to(dt[8]),
                d_bias[2 * n:].reshape(ctx.b_res_shape).to(dt[9]), None, None)


class MHCPostFunction(Function):
    """Second half: apply(x, f, H_post, M) -> y = M x + H_post f, with f = F(y_hat) of shape [B, C]."""

    @staticmethod
    def forward(ctx, x_expanded, f, H_post, M):
        from . import capi
        x = x_expanded.contiguous()
        f = f.contiguous().to(x.dtype)
        H_post, M = H_post.contiguous(), M.contiguous()
        ctx.save_for_backward(x, f, H_post, M)
        return capi.post_fwd(x, f, H_post, M)

    @staticmethod
    def backward(ctx, grad_output):
        from . import capi
        x, f, H_post, M = ctx.saved_tensors
        dx_part, d_f, dH_post, dM = capi.post_bwd(grad_output.contiguous().to(x.dtype), x, f, H_post, M)
        return dx_part, d_f, dH_post, dM


def mhc_pre(x_expanded, rmsnorm_weight, phi_pre, phi_post, phi_res, alpha_pre, alpha_post, alpha_res,
            b_pre, b_post, b_res, sinkhorn_iters=20, eps=1e-5):
    """Aggregate + RMSNorm half of the dynamic layer: returns (y_hat, H_post, M)."""
    return MHCPreFunction.apply(
        x_expanded.to(_compute_dtype(x_expanded)), rmsnorm_weight.bfloat16(), phi_pre.float(),
        phi_post.float(), phi_res.float(), alpha_pre, alpha_post, alpha_res, b_pre.float(),
        b_post.float(), b_res.float(), sinkhorn_iters, eps)


def mhc_post(x_expanded, f, H_post, M):
    """Distribute + mix half: y[i] = sum_j M[i,j] x[j] + H_post[i] f."""
    return MHCPostFunction.apply(x_expanded.to(_compute_dtype(x_expanded)), f, H_post, M)
