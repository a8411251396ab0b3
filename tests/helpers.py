"""Shared helpers for the parity tests: golden-fixture loading and the error metric."""
import glob
import os

import numpy as np
import torch

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

DYN_PARAMS = ("rmsnorm_weight", "phi_pre", "phi_post", "phi_res", "alpha_pre", "alpha_post",
              "alpha_res", "b_pre", "b_post", "b_res")
STATIC_PARAMS = ("rmsnorm_weight", "H_pre", "H_post", "H_res")


def golden_names(prefix):
    return sorted(os.path.basename(p)[:-4] for p in glob.glob(os.path.join(GOLDEN_DIR, prefix + "*.npz")))


def load_golden(name):
    """Returns a dict of float64 torch tensors (plus python ``iters`` / ``eps``)."""
    z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
    out = {}
    for k in z.files:
        if k == "iters":
            out[k] = int(z[k])
        elif k == "eps":
            out[k] = float(z[k])
        else:
            out[k] = torch.from_numpy(np.array(z[k], dtype=np.float64))
    return out


def rel_err(a, b):
    """max|a-b| / max|b|  (the metric every parity tolerance in this repo refers to)."""
    a = torch.as_tensor(a).detach().double().cpu()
    b = torch.as_tensor(b).detach().double().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    denom = max(float(b.abs().max()), 1e-30)
    return float((a - b).abs().max()) / denom


def assert_rel(a, b, tol, what=""):
    e = rel_err(a, b)
    assert e <= tol, f"{what}: relative error {e:.3e} > {tol:.1e}"
    return e
