"""GPU-side helpers of the parity tests: run the C ABI on a set of CPU tensors and hand back
results under the oracle's key names."""
import torch

from mhc.cu_b200 import capi
from mhc.cu_b200.synthetic import pack_dynamic

TOL = {torch.float32: 1e-5, torch.bfloat16: 2e-2}


def round_to(t, dtype):
    """What the kernel will actually see: the value after rounding to ``dtype``, as fp64."""
    return t.detach().to(torch.float32).to(dtype).double()


def run_dynamic(x, dy, params, iters, eps, dtype, device="cuda"):
    n = x.shape[1]
    w, phi, alpha, bias = pack_dynamic({k: v.float() for k, v in params.items()}, dtype, device)
    xd = x.to(device=device, dtype=dtype).contiguous()
    gd = dy.to(device=device, dtype=dtype).contiguous()
    y, saved = capi.dynamic_fwd(xd, w, phi, alpha, bias, iters, eps)
    dx, g = capi.dynamic_bwd(gd, xd, w, phi, alpha, bias, saved, iters, eps)
    torch.cuda.synchronize()
    out = {
        "y": y, "dx": dx, "drmsnorm_weight": g["d_rmsnorm_weight"],
        "dphi_pre": g["d_phi"][:n], "dphi_post": g["d_phi"][n:2 * n], "dphi_res": g["d_phi"][2 * n:],
        "dalpha_pre": g["d_alpha"][0], "dalpha_post": g["d_alpha"][1], "dalpha_res": g["d_alpha"][2],
        "db_pre": g["d_bias"][:n], "db_post": g["d_bias"][n:2 * n],
        "db_res": g["d_bias"][2 * n:].reshape(n, n),
    }
    return {k: v.detach().double().cpu() for k, v in out.items()}, saved


def run_static(x, dy, params, iters, eps, dtype, device="cuda"):
    xd = x.to(device=device, dtype=dtype).contiguous()
    gd = dy.to(device=device, dtype=dtype).contiguous()
    w = params["rmsnorm_weight"].to(device=device, dtype=torch.bfloat16).contiguous()
    f = lambda k: params[k].to(device=device, dtype=torch.float32).contiguous()
    y, saved = capi.static_fwd(xd, w, f("H_pre"), f("H_post"), f("H_res"), iters, eps)
    dx, g = capi.static_bwd(gd, xd, w, f("H_res"), saved, iters, eps)
    torch.cuda.synchronize()
    out = {"y": y, "dx": dx, "drmsnorm_weight": g["d_rmsnorm_weight"], "dH_pre": g["d_H_pre"],
           "dH_post": g["d_H_post"], "dH_res": g["d_H_res"]}
    return {k: v.detach().double().cpu() for k, v in out.items()}, saved


def oracle_inputs(x, dy, params, dtype, stream_rounded=("phi_pre", "phi_post", "phi_res")):
    """Inputs for the fp64 oracle: exactly what the kernels consume (x, dy and phi rounded to the
    stream dtype, rmsnorm_weight to bf16, everything else fp32)."""
    p = {}
    for k, v in params.items():
        if k == "rmsnorm_weight":
            p[k] = round_to(v, torch.bfloat16)
        elif k in stream_rounded:
            p[k] = round_to(v, dtype)
        else:
            p[k] = v.detach().float().double()
    return round_to(x, dtype), round_to(dy, dtype), p
