"""CPU oracle for the mHC layer forward + backward.

TEST INFRASTRUCTURE ONLY.  Nothing under ``mhc/`` may import this package; it is
the checker used by ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline /
reference legs of ``bench.py``.  It restates, in plain PyTorch on the CPU, the naive
mHC layer of AndreSlavescu/mHC.cu (``src/python/tests/test_layer.py:7-50`` and
``src/python/benchmarks/bench_layer.py:27-145``).

Parity is pinned: ``tests/golden/*.npz`` hold inputs, outputs and gradients produced
by importing the reference's own naive functions (``tests/golden/make_golden.py``),
and ``tests/test_oracle_golden.py`` checks this restatement against them.
"""
from .naive_mhc import (  # noqa: F401
    sinkhorn_knopp,
    rmsnorm,
    mhc_dynamic,
    mhc_dynamic_pre,
    mhc_post,
    mhc_static,
    dynamic_fwd_bwd,
    static_fwd_bwd,
)
from .closed_form import (  # noqa: F401
    sinkhorn_backward,
    dynamic_backward_closed_form,
    static_backward_closed_form,
)
