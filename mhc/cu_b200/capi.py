"""Tensor-level wrappers over the C ABI: check dtype / layout / device, allocate outputs and the
workspace with torch, pass raw pointers and the current CUDA stream to libmhc_b200.so.

These are thin on purpose: one Python function per entry point of include/mhc_b200.h, same
argument meaning.  Parity tests call these; ``mhc.ops`` builds the autograd Functions on them.
"""
from __future__ import annotations

import torch

from . import _lib as L


def _dtype_tag(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return L.F32
    if t.dtype == torch.bfloat16:
        return L.BF16
    raise TypeError(f"streams must be float32 or bfloat16, got {t.dtype}")


def _chk(t: torch.Tensor, name: str, dtype=None, shape=None):
    if not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise TypeError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and tuple(t.shape) != tuple(shape):
        raise ValueError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")
    return t


def _ptr(t):
    return None if t is None else t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def workspace_bytes(op: int, B: int, n: int, C: int, iters: int, dtype_tag: int) -> int:
    v = L.lib().mhc_workspace_bytes(op, B, n, C, iters, dtype_tag)
    if v == (1 << 64) - 1:
        raise ValueError(f"bad problem size B={B} n={n} C={C} iters={iters}")
    return v


# Debug aid for the parity tests: when set, every buffer this module allocates (outputs, saved
# tensors, workspace) starts as all-ones bytes (NaN in every floating type), so a kernel that reads
# a slot nobody wrote shows up in the results instead of depending on what the allocator returns.
POISON = False


def _empty(*shape, **kw):
    t = torch.empty(*shape, **kw)
    if POISON and t.numel():
        t.view(torch.uint8).fill_(0xFF)
    return t


def _empty_like(t):
    return _empty(t.shape, dtype=t.dtype, device=t.device)


def _workspace(nbytes: int, device, given=None):
    if given is not None:
        if given.numel() * given.element_size() < nbytes:
            raise ValueError("workspace too small")
        return given
    return _empty(max(nbytes, 16), dtype=torch.uint8, device=device)


def dynamic_fwd(x, rmsnorm_weight, phi, alpha, bias, iters, eps, *, y=None, workspace=None):
    """mhc_dynamic_fwd.  x [B,n,C] fp32|bf16; rmsnorm_weight [C] bf16; phi [K,nC] same dtype as x
    (rows pre, post, res); alpha [3] fp32; bias [K] fp32.  Returns (y, saved) where saved holds the
    fp32 tensors rms, rms_h, H_pre, H_post, M, proj, sk_den."""
    B, n, C = x.shape
    K = 2 * n + n * n
    tag = _dtype_tag(x)
    _chk(x, "x")
    _chk(rmsnorm_weight, "rmsnorm_weight", torch.bfloat16, (C,))
    _chk(phi, "phi", x.dtype, (K, n * C))
    _chk(alpha, "alpha", torch.float32, (3,))
    _chk(bias, "bias", torch.float32, (K,))
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    y = _empty_like(x) if y is None else _chk(y, "y", x.dtype, x.shape)
    saved = {
        "rms": _empty(B, **f32), "rms_h": _empty(B, **f32),
        "H_pre": _empty(B, n, **f32), "H_post": _empty(B, n, **f32),
        "M": _empty(B, n, n, **f32), "proj": _empty(B, K, **f32),
        "sk_den": _empty(B, 2 * int(iters), 4 if n <= 4 else 8, **f32),
    }
    nbytes = workspace_bytes(L.OP_DYNAMIC_FWD, B, n, C, iters, tag)
    ws = _workspace(nbytes, dev, workspace)
    st = L.lib().mhc_dynamic_fwd(
        _ptr(y), _ptr(saved["rms"]), _ptr(saved["rms_h"]), _ptr(saved["H_pre"]), _ptr(saved["H_post"]),
        _ptr(saved["M"]), _ptr(saved["proj"]), _ptr(saved["sk_den"]), _ptr(x), _ptr(rmsnorm_weight),
        _ptr(phi), _ptr(alpha), _ptr(bias), B, n, C, int(iters), float(eps), tag, _ptr(ws),
        ws.numel(), _stream())
    L.check(st, "mhc_dynamic_fwd")
    return y, saved


def dynamic_bwd(dy, x, rmsnorm_weight, phi, alpha, bias, saved, iters, eps, *, grads=None,
                dx=None, workspace=None):
    """mhc_dynamic_bwd.  ``grads`` may supply preallocated fp32 outputs (keys d_rmsnorm_weight [C],
    d_phi [K,nC], d_alpha [3], d_bias [K]) — e.g. slices of one flat all-reduce bucket.
    Returns (dx, grads)."""
    B, n, C = x.shape
    K = 2 * n + n * n
    tag = _dtype_tag(x)
    _chk(x, "x")
    _chk(dy, "dy", x.dtype, x.shape)
    _chk(rmsnorm_weight, "rmsnorm_weight", torch.bfloat16, (C,))
    _chk(phi, "phi", x.dtype, (K, n * C))
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    if grads is None:
        grads = {"d_rmsnorm_weight": _empty(C, **f32), "d_phi": _empty(K, n * C, **f32),
                 "d_alpha": _empty(3, **f32), "d_bias": _empty(K, **f32)}
    _chk(grads["d_rmsnorm_weight"], "d_rmsnorm_weight", torch.float32, (C,))
    _chk(grads["d_phi"], "d_phi", torch.float32, (K, n * C))
    _chk(grads["d_alpha"], "d_alpha", torch.float32, (3,))
    _chk(grads["d_bias"], "d_bias", torch.float32, (K,))
    dx = _empty_like(x) if dx is None else _chk(dx, "dx", x.dtype, x.shape)
    nbytes = workspace_bytes(L.OP_DYNAMIC_BWD, B, n, C, iters, tag)
    ws = _workspace(nbytes, dev, workspace)
    st = L.lib().mhc_dynamic_bwd(
        _ptr(dx), _ptr(grads["d_rmsnorm_weight"]), _ptr(grads["d_phi"]), _ptr(grads["d_alpha"]),
        _ptr(grads["d_bias"]), _ptr(dy), _ptr(x), _ptr(rmsnorm_weight), _ptr(phi), _ptr(alpha),
        _ptr(bias), _ptr(saved["rms"]), _ptr(saved["rms_h"]), _ptr(saved["H_pre"]),
        _ptr(saved["H_post"]), _ptr(saved["M"]), _ptr(saved["proj"]), _ptr(saved.get("sk_den")),
        B, n, C, int(iters), float(eps), tag, _ptr(ws), ws.numel(), _stream())
    L.check(st, "mhc_dynamic_bwd")
    return dx, grads


def static_fwd(x, rmsnorm_weight, H_pre, H_post, H_res, iters, eps, *, inference=False, y=None,
               workspace=None):
    """mhc_static_fwd.  H_pre [n], H_post [n], H_res [n,n]: raw fp32 parameters.
    Returns (y, saved) with saved = rms, H_pre_act, H_post_act, M; with ``inference=True`` nothing is
    saved (the intermediates live in the workspace) and saved is None."""
    B, n, C = x.shape
    tag = _dtype_tag(x)
    _chk(x, "x")
    _chk(rmsnorm_weight, "rmsnorm_weight", torch.bfloat16, (C,))
    _chk(H_pre, "H_pre", torch.float32, (n,))
    _chk(H_post, "H_post", torch.float32, (n,))
    _chk(H_res, "H_res", torch.float32, (n, n))
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    y = _empty_like(x) if y is None else _chk(y, "y", x.dtype, x.shape)
    saved = None
    if not inference:
        saved = {"rms": _empty(B, **f32), "H_pre_act": _empty(n, **f32),
                 "H_post_act": _empty(n, **f32), "M": _empty(n, n, **f32)}
    nbytes = workspace_bytes(L.OP_STATIC_FWD, B, n, C, iters, tag)
    ws = _workspace(nbytes, dev, workspace)
    g = (lambda k: _ptr(saved[k])) if saved is not None else (lambda k: None)
    st = L.lib().mhc_static_fwd(
        _ptr(y), g("rms"), g("H_pre_act"), g("H_post_act"), g("M"), _ptr(x), _ptr(rmsnorm_weight),
        _ptr(H_pre), _ptr(H_post), _ptr(H_res), B, n, C, int(iters), float(eps), tag, _ptr(ws),
        ws.numel(), _stream())
    L.check(st, "mhc_static_fwd")
    return y, saved


def static_bwd(dy, x, rmsnorm_weight, H_res, saved, iters, eps, *, grads=None, dx=None,
               workspace=None):
    """mhc_static_bwd.  Returns (dx, grads) with fp32 grads d_rmsnorm_weight [C], d_H_pre [n],
    d_H_post [n], d_H_res [n,n] (w.r.t. the raw parameters)."""
    B, n, C = x.shape
    tag = _dtype_tag(x)
    _chk(x, "x")
    _chk(dy, "dy", x.dtype, x.shape)
    _chk(rmsnorm_weight, "rmsnorm_weight", torch.bfloat16, (C,))
    _chk(H_res, "H_res", torch.float32, (n, n))
    dev = x.device
    f32 = dict(dtype=torch.float32, device=dev)
    if grads is None:
        grads = {"d_rmsnorm_weight": _empty(C, **f32), "d_H_pre": _empty(n, **f32),
                 "d_H_post": _empty(n, **f32), "d_H_res": _empty(n, n, **f32)}
    dx = _empty_like(x) if dx is None else _chk(dx, "dx", x.dtype, x.shape)
    nbytes = workspace_bytes(L.OP_STATIC_BWD, B, n, C, iters, tag)
    ws = _workspace(nbytes, dev, workspace)
    st = L.lib().mhc_static_bwd(
        _ptr(dx), _ptr(grads["d_rmsnorm_weight"]), _ptr(grads["d_H_pre"]), _ptr(grads["d_H_post"]),
        _ptr(grads["d_H_res"]), _ptr(dy), _ptr(x), _ptr(rmsnorm_weight), _ptr(H_res),
        _ptr(saved["rms"]), _ptr(saved["H_pre_act"]), _ptr(saved["H_post_act"]), _ptr(saved["M"]),
        B, n, C, int(iters), float(eps), tag, _ptr(ws), ws.numel(), _stream())
    L.check(st, "mhc_static_bwd")
    return dx, grads


def dynamic_pre_fwd(x, rmsnorm_weight, phi, alpha, bias, iters, eps):
    """mhc_dynamic_pre_fwd: first half of the split layer.  Returns (y_hat [B,C], saved) with saved
    holding rms, rms_h, H_pre, H_post, M, proj (fp32)."""
    tag = _dtype_tag(x)
    _chk(x, "x", x.dtype)
    B, n, C = x.shape
    K = 2 * n + n * n
    f32 = dict(dtype=torch.float32, device=x.device)
    y_hat = _empty(B, C, dtype=x.dtype, device=x.device)
    saved = {"rms": _empty(B, **f32), "rms_h": _empty(B, **f32), "H_pre": _empty(B, n, **f32),
             "H_post": _empty(B, n, **f32), "M": _empty(B, n, n, **f32), "proj": _empty(B, K, **f32)}
    ws = _workspace(workspace_bytes(L.OP_DYNAMIC_FWD, B, n, C, iters, tag), x.device)
    st = L.lib().mhc_dynamic_pre_fwd(
        _ptr(y_hat), _ptr(saved["rms"]), _ptr(saved["rms_h"]), _ptr(saved["H_pre"]),
        _ptr(saved["H_post"]), _ptr(saved["M"]), _ptr(saved["proj"]), _ptr(x), _ptr(rmsnorm_weight),
        _ptr(phi), _ptr(alpha), _ptr(bias), B, n, C, int(iters), float(eps), tag, _ptr(ws),
        ws.numel(), _stream())
    L.check(st, "mhc_dynamic_pre_fwd")
    return y_hat, saved


def post_fwd(x, f, H_post, M):
    """mhc_post_fwd: y = M x + H_post f."""
    tag = _dtype_tag(x)
    B, n, C = x.shape
    _chk(f, "f", x.dtype, (B, C))
    y = _empty_like(x)
    st = L.lib().mhc_post_fwd(_ptr(y), _ptr(x), _ptr(f), _ptr(H_post), _ptr(M), B, n, C, tag,
                              _stream())
    L.check(st, "mhc_post_fwd")
    return y


def post_bwd(dy, x, f, H_post, M):
    """mhc_post_bwd: returns (dx_part, d_f, dH_post, dM)."""
    tag = _dtype_tag(x)
    B, n, C = x.shape
    _chk(dy, "dy", x.dtype, x.shape)
    f32 = dict(dtype=torch.float32, device=x.device)
    dx_part, d_f = _empty_like(x), _empty_like(f)
    dH_post, dM = _empty(B, n, **f32), _empty(B, n, n, **f32)
    st = L.lib().mhc_post_bwd(_ptr(dx_part), _ptr(d_f), _ptr(dH_post), _ptr(dM), _ptr(dy), _ptr(x),
                              _ptr(f), _ptr(H_post), _ptr(M), B, n, C, tag, _stream())
    L.check(st, "mhc_post_bwd")
    return dx_part, d_f, dH_post, dM


def dynamic_pre_bwd(d_y_hat, dH_post, dM, x, rmsnorm_weight, phi, alpha, bias, saved, iters, eps):
    """mhc_dynamic_pre_bwd: returns (dx, grads) with grads = d_rmsnorm_weight, d_phi, d_alpha, d_bias."""
    tag = _dtype_tag(x)
    B, n, C = x.shape
    K = 2 * n + n * n
    _chk(d_y_hat, "d_y_hat", x.dtype, (B, C))
    f32 = dict(dtype=torch.float32, device=x.device)
    grads = {"d_rmsnorm_weight": _empty(C, **f32), "d_phi": _empty(K, n * C, **f32),
             "d_alpha": _empty(3, **f32), "d_bias": _empty(K, **f32)}
    dx = _empty_like(x)
    ws = _workspace(workspace_bytes(L.OP_DYNAMIC_PRE_BWD, B, n, C, iters, tag), x.device)
    st = L.lib().mhc_dynamic_pre_bwd(
        _ptr(dx), _ptr(grads["d_rmsnorm_weight"]), _ptr(grads["d_phi"]), _ptr(grads["d_alpha"]),
        _ptr(grads["d_bias"]), _ptr(d_y_hat), _ptr(dH_post), _ptr(dM), _ptr(x), _ptr(rmsnorm_weight),
        _ptr(phi), _ptr(alpha), _ptr(bias), _ptr(saved["rms"]), _ptr(saved["rms_h"]),
        _ptr(saved["H_pre"]), _ptr(saved["H_post"]), _ptr(saved["proj"]), B, n, C, int(iters),
        float(eps), tag, _ptr(ws), ws.numel(), _stream())
    L.check(st, "mhc_dynamic_pre_bwd")
    return dx, grads


def _is_rect(inp):
    """A single 2-D matrix that the batched square kernels (n <= 32) do not cover."""
    return inp.dim() == 2 and (inp.shape[0] != inp.shape[1] or inp.shape[0] > 32)


def sinkhorn_fwd(inp, iters, eps):
    """mhc_sinkhorn_fwd on fp32 [n,n] / [batch,n,n] (n <= 32), mhc_sinkhorn_rect_fwd on one [M,N]
    matrix with M, N <= 128."""
    _chk(inp, "inp", torch.float32)
    if _is_rect(inp):
        M, N = inp.shape
        out = _empty_like(inp)
        st = L.lib().mhc_sinkhorn_rect_fwd(_ptr(out), _ptr(inp), M, N, int(iters), float(eps),
                                           _stream())
        L.check(st, "mhc_sinkhorn_rect_fwd")
        return out
    if inp.dim() not in (2, 3) or inp.shape[-1] != inp.shape[-2]:
        raise ValueError("sinkhorn expects one [M,N] matrix (M, N <= 128) or square [batch,n,n]")
    n = inp.shape[-1]
    batch = inp.shape[0] if inp.dim() == 3 else 1
    out = _empty_like(inp)
    st = L.lib().mhc_sinkhorn_fwd(_ptr(out), _ptr(inp), batch, n, int(iters), float(eps), _stream())
    L.check(st, "mhc_sinkhorn_fwd")
    return out


def sinkhorn_bwd(grad_out, inp, iters, eps):
    """mhc_sinkhorn_bwd: gradient w.r.t. ``inp`` of sinkhorn_fwd(inp)."""
    _chk(inp, "inp", torch.float32)
    _chk(grad_out, "grad_out", torch.float32, inp.shape)
    if _is_rect(inp):
        M, N = inp.shape
        d_inp = _empty_like(inp)
        nbytes = workspace_bytes(L.OP_SINKHORN_RECT_BWD, M, N, 0, iters, L.F32)
        ws = _workspace(nbytes, inp.device)
        st = L.lib().mhc_sinkhorn_rect_bwd(_ptr(d_inp), _ptr(grad_out), _ptr(inp), M, N, int(iters),
                                           float(eps), _ptr(ws), ws.numel(), _stream())
        L.check(st, "mhc_sinkhorn_rect_bwd")
        return d_inp
    n = inp.shape[-1]
    batch = inp.shape[0] if inp.dim() == 3 else 1
    d_inp = _empty_like(inp)
    nbytes = workspace_bytes(L.OP_SINKHORN_BWD, batch, n, 0, iters, L.F32)
    ws = _workspace(nbytes, inp.device)
    st = L.lib().mhc_sinkhorn_bwd(_ptr(d_inp), _ptr(grad_out), _ptr(inp), batch, n, int(iters),
                                  float(eps), _ptr(ws), ws.numel(), _stream())
    L.check(st, "mhc_sinkhorn_bwd")
    return d_inp


def rmsnorm_fwd(inp, weight, eps):
    """mhc_rmsnorm_fwd on bf16 [B,C]; returns (out bf16, rms fp32 [B])."""
    _chk(inp, "inp", torch.bfloat16)
    B, Cc = inp.shape
    _chk(weight, "weight", torch.bfloat16, (Cc,))
    out = _empty_like(inp)
    rms = _empty(B, dtype=torch.float32, device=inp.device)
    st = L.lib().mhc_rmsnorm_fwd(_ptr(out), _ptr(rms), _ptr(inp), _ptr(weight), B, Cc, float(eps), _stream())
    L.check(st, "mhc_rmsnorm_fwd")
    return out, rms


def rmsnorm_bwd(grad_out, inp, weight, rms):
    """mhc_rmsnorm_bwd; returns (d_inp bf16 [B,C], d_weight fp32 [C])."""
    _chk(inp, "inp", torch.bfloat16)
    B, Cc = inp.shape
    _chk(grad_out, "grad_out", torch.bfloat16, inp.shape)
    _chk(weight, "weight", torch.bfloat16, (Cc,))
    _chk(rms, "rms", torch.float32, (B,))
    d_inp = _empty_like(inp)
    d_w = _empty(Cc, dtype=torch.float32, device=inp.device)
    nbytes = workspace_bytes(L.OP_RMSNORM_BWD, B, 1, Cc, 0, L.BF16)
    ws = _workspace(nbytes, inp.device)
    st = L.lib().mhc_rmsnorm_bwd(_ptr(d_inp), _ptr(d_w), _ptr(grad_out), _ptr(inp), _ptr(weight),
                                 _ptr(rms), B, Cc, _ptr(ws), ws.numel(), _stream())
    L.check(st, "mhc_rmsnorm_bwd")
    return d_inp, d_w
