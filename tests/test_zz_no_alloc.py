"""mhc_sinkhorn_bwd_noalloc — the one entry point that needs no workspace from its caller.

It exists for callers that cannot allocate device memory where they run (a plug-in in a host that
keeps all device memory to itself, code that must stay clear of cudaMalloc).  Its scratch is a
fixed array inside the library, so this test checks three things through the C ABI: the result
equals that of the workspace-taking mhc_sinkhorn_bwd, it still does on a second call that finds
the first call's leftovers in the array, and a problem larger than the array is refused with
MHC_ERR_LIMIT instead of being run.  The file sorts last on purpose, so a run that stops at the
first failure has already been through every other test.
"""
import pytest
import torch

from mhc.cu_b200 import _lib as L
from mhc.cu_b200 import capi

pytestmark = pytest.mark.gpu


def _noalloc(grad, inp, iters, eps):
    out = torch.empty_like(inp)
    n = inp.shape[-1]
    batch = inp.shape[0] if inp.dim() == 3 else 1
    st = L.lib().mhc_sinkhorn_bwd_noalloc(out.data_ptr(), grad.data_ptr(), inp.data_ptr(), batch, n,
                                          iters, eps, torch.cuda.current_stream().cuda_stream)
    return st, out


def test_noalloc_matches_workspace_entry_point_twice():
    gen = torch.Generator().manual_seed(11)
    # two different problems back to back: the second one runs over the first one's leftovers
    for batch, n, iters in ((64, 4, 20), (9, 8, 12)):
        E = torch.exp(torch.randn(batch, n, n, generator=gen) * 0.5).cuda()
        dM = torch.randn(batch, n, n, generator=gen).cuda()
        ref = capi.sinkhorn_bwd(dM, E, iters, 1e-6)
        st, got = _noalloc(dM, E, iters, 1e-6)
        assert st == 0
        torch.cuda.synchronize()
        err = float((got - ref).abs().max() / ref.abs().max())
        assert err <= 1e-5, err
    # and the first problem once more, now after a different-sized call
    E = torch.exp(torch.randn(64, 4, 4, generator=gen) * 0.5).cuda()
    dM = torch.randn(64, 4, 4, generator=gen).cuda()
    ref = capi.sinkhorn_bwd(dM, E, 20, 1e-6)
    st, got = _noalloc(dM, E, 20, 1e-6)
    assert st == 0
    torch.cuda.synchronize()
    assert float((got - ref).abs().max() / ref.abs().max()) <= 1e-5


def test_noalloc_refuses_what_does_not_fit():
    cap = L.lib().mhc_sinkhorn_bwd_noalloc_capacity()
    assert cap == 1 << 20
    batch, n, iters = 4096, 32, 20          # needs far more than the built-in array
    need = capi.workspace_bytes(L.OP_SINKHORN_BWD, batch, n, 0, iters, L.F32)
    assert need > cap
    x = torch.ones(batch, n, n, device="cuda")
    out = torch.full_like(x, 7.0)
    st = L.lib().mhc_sinkhorn_bwd_noalloc(out.data_ptr(), x.data_ptr(), x.data_ptr(), batch, n, iters,
                                          1e-6, torch.cuda.current_stream().cuda_stream)
    assert st == 8                           # MHC_ERR_LIMIT
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())          # nothing ran
