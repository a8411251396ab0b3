"""Stand-alone Sinkhorn-Knopp and RMSNorm ops, and the C ABI's argument checking, on the GPU."""
import pytest
import torch

import oracle
from helpers import assert_rel, golden_names, load_golden
from mhc.cu_b200 import _lib as L
from mhc.cu_b200 import capi

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("name", golden_names("sinkhorn"))
def test_sinkhorn_golden(name):
    g = load_golden(name)
    inp = g["inp"].float().cuda()
    out = capi.sinkhorn_fwd(inp, g["iters"], g["eps"])
    assert_rel(out, g["out"], 1e-5, "sinkhorn forward")
    d = capi.sinkhorn_bwd(g["grad_out"].float().cuda(), inp, g["iters"], g["eps"])
    assert_rel(d, g["grad_inp"], 1e-5, "sinkhorn backward")


def test_sinkhorn_doubly_stochastic_32():
    """32x32, 20 iterations: rows and columns sum to 1 within 1e-5
    (src/python/tests/test_ops.py:7-18 of the reference)."""
    torch.manual_seed(42)
    inp = torch.rand(32, 32, device="cuda") + 0.1
    out = capi.sinkhorn_fwd(inp, 20, 1e-8)
    assert float((out.sum(1) - 1).abs().max()) < 1e-5
    assert float((out.sum(0) - 1).abs().max()) < 1e-5
    assert bool((out >= 0).all())


@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 8, 13, 16, 32])
def test_sinkhorn_batched_sizes(n):
    gen = torch.Generator().manual_seed(n)
    E = torch.exp(torch.randn(37, n, n, generator=gen) * 0.5)
    dM = torch.randn(37, n, n, generator=gen)
    out = capi.sinkhorn_fwd(E.cuda(), 20, 1e-6)
    assert_rel(out, oracle.sinkhorn_knopp(E.double(), 20, 1e-6), 1e-5, "fwd")
    d = capi.sinkhorn_bwd(dM.cuda(), E.cuda(), 20, 1e-6)
    assert_rel(d, oracle.sinkhorn_backward(dM.double(), E.double(), 20, 1e-6), 1e-5, "bwd")


def test_sinkhorn_extremes_finite():
    """x1000 and 1e-6-sized inputs stay finite (test_ops.py:62-77 of the reference)."""
    torch.manual_seed(0)
    for inp, it in ((torch.rand(32, 32) * 1000, 50), (torch.rand(32, 32) * 1e-6 + 1e-8, 20)):
        out = capi.sinkhorn_fwd(inp.cuda(), it, 1e-8)
        assert bool(torch.isfinite(out).all())


@pytest.mark.parametrize("B,C", [(8, 128), (16, 64), (128, 4096), (3, 100), (5, 10240)])
def test_rmsnorm(B, C):
    gen = torch.Generator().manual_seed(C)
    x = (torch.randn(B, C, generator=gen) * 0.5).bfloat16()
    w = (1 + 0.25 * torch.randn(C, generator=gen)).bfloat16()
    g = torch.randn(B, C, generator=gen).bfloat16()
    out, rms = capi.rmsnorm_fwd(x.cuda(), w.cuda(), 1e-5)
    xd = x.double().requires_grad_(True)
    wd = w.double().requires_grad_(True)
    ref = oracle.rmsnorm(xd, wd, 1e-5)
    assert out.dtype == torch.bfloat16
    assert_rel(out, ref, 1e-2, "rmsnorm out")            # bf16 output rounding (reference: 1e-2)
    dxr, dwr = torch.autograd.grad(ref, [xd, wd], grad_outputs=g.double())
    d_inp, d_w = capi.rmsnorm_bwd(g.cuda(), x.cuda(), w.cuda(), rms)
    assert_rel(d_inp, dxr, 2e-2, "rmsnorm d_inp")
    assert_rel(d_w, dwr, 2e-2, "rmsnorm d_weight")


def test_abi_rejects_bad_arguments():
    """Bad requests come back as status codes; nothing is launched and the process lives."""
    h = L.lib()
    x = torch.zeros(2, 4, 64, device="cuda")
    ws = torch.zeros(1 << 16, dtype=torch.uint8, device="cuda")
    p = x.data_ptr()
    args = lambda n, dtype, ptr=p, wsb=ws.numel(): (
        ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, ptr, 2, n, 64, 20, 1e-5, dtype,
        ws.data_ptr(), wsb, None)
    assert h.mhc_dynamic_fwd(*args(0, 0)) == 2          # n out of range
    assert h.mhc_dynamic_fwd(*args(33, 0)) == 2
    assert h.mhc_dynamic_fwd(*args(4, 5)) == 3          # dtype tag
    assert h.mhc_dynamic_fwd(*args(4, 0, ptr=None)) == 1
    assert h.mhc_dynamic_fwd(*args(4, 0, ptr=p + 4)) == 4
    assert h.mhc_dynamic_fwd(*args(4, 0, wsb=8)) == 5
    assert b"aligned" in h.mhc_status_string(4)
    with pytest.raises(RuntimeError):
        capi.dynamic_fwd(torch.zeros(2, 4, 64), None, None, None, None, 20, 1e-5)  # CPU tensor


@pytest.mark.parametrize("M,N", [(33, 33), (64, 64), (128, 128), (100, 80), (5, 128), (128, 3),
                                 (1, 7), (7, 1), (48, 96)])
def test_sinkhorn_single_matrix_up_to_128(M, N):
    """One [M, N] matrix beyond the batched square kernels: the shape range of the reference's
    single-matrix op (src/csrc/kernels/sinkhorn_knopp.cuh:423-459), rectangular included, forward
    and exact backward against the oracle (its backward is checked against autograd on the CPU)."""
    gen = torch.Generator().manual_seed(1000 * M + N)
    E = torch.exp(torch.randn(M, N, generator=gen) * 0.5)
    dM = torch.randn(M, N, generator=gen)
    out = capi.sinkhorn_fwd(E.cuda(), 20, 1e-6)
    assert_rel(out, oracle.sinkhorn_knopp(E.double(), 20, 1e-6), 1e-5, "fwd")
    d = capi.sinkhorn_bwd(dM.cuda(), E.cuda(), 20, 1e-6)
    assert_rel(d, oracle.sinkhorn_backward(dM.double(), E.double(), 20, 1e-6), 1e-5, "bwd")


def test_sinkhorn_single_matrix_through_autograd():
    """mhc.sinkhorn_knopp on a 64 x 64 and on a 100 x 80 matrix, gradient through the extension."""
    import mhc
    for M, N in ((64, 64), (100, 80)):
        gen = torch.Generator().manual_seed(M)
        E = torch.exp(torch.randn(M, N, generator=gen) * 0.5)
        dM = torch.randn(M, N, generator=gen)
        inp = E.cuda().requires_grad_(True)
        out = mhc.sinkhorn_knopp(inp, 20, 1e-6)
        out.backward(dM.cuda())
        assert_rel(out.detach(), oracle.sinkhorn_knopp(E.double(), 20, 1e-6), 1e-5, "fwd")
        assert_rel(inp.grad, oracle.sinkhorn_backward(dM.double(), E.double(), 20, 1e-6), 1e-5, "bwd")


def test_sinkhorn_single_matrix_rejects_large():
    big = torch.rand(129, 4, device="cuda")
    with pytest.raises(Exception):
        capi.sinkhorn_fwd(big, 5, 1e-6)
