#!/usr/bin/env python3
"""Generate the golden vectors under tests/golden/ from the reference's own naive code.

Run in a container that has a checkout of the reference (pass its path with --reference):

    python tests/golden/make_golden.py [--reference /path/to/mHC.cu]

It imports, unmodified and on the CPU, the reference's
  * ``_naive_mhc_dynamic``            (src/python/tests/test_layer.py:7-50)
  * ``NaiveMHCLayer``                 (src/python/benchmarks/bench_layer.py:27-71)
  * ``NaiveMHCLayerDynamic``          (src/python/benchmarks/bench_layer.py:74-145)
(both files import ``mhc`` only inside function bodies, so no CUDA extension is needed),
feeds them seeded inputs, takes gradients with autograd, and stores inputs, outputs and
gradients as float64 arrays in one ``.npz`` per case.  Inputs are drawn in float32 and then
widened, so a float32 consumer sees exactly the same numbers.

The fixtures are what pins ``oracle/`` to the reference; the GPU box has no reference
checkout, so they are committed.
"""
import argparse
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _randn(gen, *shape, scale=1.0, shift=0.0):
    return (torch.randn(*shape, generator=gen, dtype=torch.float32) * scale + shift).double()


def _bf16_exact(t):
    """The layer keeps rmsnorm_weight as a bf16 parameter: use values bf16 can hold exactly."""
    return t.float().bfloat16().double()


def _save(name, arrays):
    out = {k: (v.detach().numpy() if torch.is_tensor(v) else np.asarray(v)) for k, v in arrays.items()}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print(f"wrote {name}.npz  ({', '.join(sorted(out))})")


def dynamic_case(ref_fn, name, seed, B, n, C, iters, eps, alpha, bias_scale, w_random):
    gen = torch.Generator().manual_seed(seed)
    nC = n * C
    leaves = {
        "x": _randn(gen, B, n, C),
        "rmsnorm_weight": _bf16_exact(_randn(gen, C, scale=0.25, shift=1.0)) if w_random else torch.ones(C).double(),
        "phi_pre": _randn(gen, n, nC, scale=0.02),
        "phi_post": _randn(gen, n, nC, scale=0.02),
        "phi_res": _randn(gen, n * n, nC, scale=0.02),
        "alpha_pre": torch.tensor(alpha[0]).float().double(),
        "alpha_post": torch.tensor(alpha[1]).float().double(),
        "alpha_res": torch.tensor(alpha[2]).float().double(),
        "b_pre": _randn(gen, n, scale=bias_scale),
        "b_post": _randn(gen, n, scale=bias_scale),
        "b_res": _randn(gen, n, n, scale=bias_scale),
    }
    dy = _randn(gen, B, n, C)
    order = ["x", "rmsnorm_weight", "phi_pre", "phi_post", "phi_res", "alpha_pre", "alpha_post",
             "alpha_res", "b_pre", "b_post", "b_res"]
    args = [leaves[k].clone().requires_grad_(True) for k in order]
    y = ref_fn(*args, iters, eps)
    grads = torch.autograd.grad(y, args, grad_outputs=dy)
    out = dict(leaves)
    out.update({"dy": dy, "y": y, "iters": iters, "eps": eps})
    for k, g in zip(order, grads):
        out["d" + k] = g
    _save(name, out)


def dynamic_class_case(cls, name, seed, B, n, C, iters, eps):
    """Goes through the reference's nn.Module (phi stored transposed, [nC, n])."""
    torch.manual_seed(seed)
    layer = cls(C, n, iters, eps, alpha_init=0.01).double()
    gen = torch.Generator().manual_seed(seed + 1)
    x = _randn(gen, B, n, C).requires_grad_(True)
    dy = _randn(gen, B, n, C)
    y = layer(x)
    y.backward(dy)
    out = {"x": x.detach(), "dy": dy, "y": y, "dx": x.grad, "iters": iters, "eps": eps}
    for k, p in layer.named_parameters():
        v, g = p.detach(), p.grad
        if k.startswith("phi"):            # to the MHCLayer layout [rows, nC]
            v, g = v.t().contiguous(), g.t().contiguous()
        out[k] = v
        out["d" + k] = g
    _save(name, out)


def static_case(cls, name, seed, B, n, C, iters, eps):
    torch.manual_seed(seed)
    layer = cls(C, n, iters, eps).double()
    gen = torch.Generator().manual_seed(seed + 1)
    with torch.no_grad():
        layer.H_pre.copy_(_randn(gen, n))
        layer.H_post.copy_(_randn(gen, n))
        layer.H_res.copy_(_randn(gen, n, n))
        layer.rmsnorm_weight.copy_(_bf16_exact(_randn(gen, C, scale=0.25, shift=1.0)))
    x = _randn(gen, B, n, C).requires_grad_(True)
    dy = _randn(gen, B, n, C)
    y = layer(x)
    y.backward(dy)
    out = {"x": x.detach(), "dy": dy, "y": y, "dx": x.grad, "iters": iters, "eps": eps}
    for k, p in layer.named_parameters():
        out[k] = p.detach()
        out["d" + k] = p.grad
    _save(name, out)


def sinkhorn_case(cls, name, seed, n, iters, eps):
    """The reference's Sinkhorn takes the log-domain matrix and exponentiates it
    (bench_layer.py:112-117); feed it log(A) so the fixture is Sinkhorn(A)."""
    gen = torch.Generator().manual_seed(seed)
    A = (torch.rand(n, n, generator=gen, dtype=torch.float32) + 0.1).double()
    layer = cls(8, n, iters, eps).double()
    logA = torch.log(A).requires_grad_(True)
    out = layer.sinkhorn_knopp(logA)
    dM = _randn(gen, n, n)
    (dlog,) = torch.autograd.grad(out, logA, grad_outputs=dM)
    # d/dA = d/dlogA / A
    _save(name, {"inp": torch.exp(logA.detach()), "out": out, "grad_out": dM,
                 "grad_inp": dlog / torch.exp(logA.detach()), "iters": iters, "eps": eps})


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get("MHC_REFERENCE_CHECKOUT",
                                                          os.path.join(os.sep, "root", "reference")))
    args = ap.parse_args()
    tl = _load(os.path.join(args.reference, "src/python/tests/test_layer.py"), "ref_test_layer")
    bl = _load(os.path.join(args.reference, "src/python/benchmarks/bench_layer.py"), "ref_bench_layer")
    fn = tl._naive_mhc_dynamic

    # the reference test's own shape (test_layer.py:145-193): B=2, n=4, C=16, 3 iterations
    dynamic_case(fn, "dyn_reftest_b2_n4_c16_t3", 42, 2, 4, 16, 3, 1e-5, (0.01, 0.01, 0.01), 0.0, False)
    # coefficients that differ strongly between tokens
    dynamic_case(fn, "dyn_b5_n4_c24_t20", 1, 5, 4, 24, 20, 1e-5, (0.7, -0.4, 0.9), 0.5, True)
    dynamic_case(fn, "dyn_b3_n8_c16_t20", 2, 3, 8, 16, 20, 1e-6, (0.5, 0.6, 0.4), 0.3, True)
    dynamic_case(fn, "dyn_b2_n2_c8_t5", 3, 2, 2, 8, 5, 1e-5, (0.3, 0.3, 0.3), 0.2, True)
    dynamic_case(fn, "dyn_b2_n16_c8_t20", 4, 2, 16, 8, 20, 1e-6, (0.5, 0.5, 0.5), 0.2, True)
    dynamic_class_case(bl.NaiveMHCLayerDynamic, "dyncls_b4_n4_c32_t20", 5, 4, 4, 32, 20, 1e-5)
    static_case(bl.NaiveMHCLayer, "static_b6_n4_c32_t20", 6, 6, 4, 32, 20, 1e-5)
    static_case(bl.NaiveMHCLayer, "static_b3_n8_c16_t20", 7, 3, 8, 16, 20, 1e-5)
    sinkhorn_case(bl.NaiveMHCLayerDynamic, "sinkhorn_32x32_t20", 8, 32, 20, 1e-8)
    sinkhorn_case(bl.NaiveMHCLayerDynamic, "sinkhorn_4x4_t20", 9, 4, 20, 1e-5)


if __name__ == "__main__":
    sys.exit(main())
