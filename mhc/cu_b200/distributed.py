"""Data parallelism for the mHC layer: tokens are sharded across ranks, parameters replicated.

The forward needs no communication.  The backward's parameter gradients (sums over tokens) are
written by the kernels straight into ONE flat fp32 bucket per layer, laid out
``d_phi [K, nC] | d_bias [K] | d_alpha [3] (+1 pad) | d_rmsnorm_weight [C]``,
which is all-reduced once per step (NCCL on GPUs; any torch.distributed backend works, the
CPU tests use gloo).  The reference has no multi-GPU support at all (no NCCL / torch.distributed
call site anywhere in AndreSlavescu/mHC.cu).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_bounds(total: int, rank: int, world: int):
    """Contiguous [begin, end) of ``total`` tokens owned by ``rank``; sizes differ by at most one."""
    base, rem = divmod(total, world)
    begin = rank * base + min(rank, rem)
    return begin, begin + base + (1 if rank < rem else 0)


class GradBucket:
    """Flat fp32 gradient buffer of one dynamic-H layer with typed views into it."""

    def __init__(self, n: int, C: int, device):
        self.n, self.C = n, C
        K, nC = 2 * n + n * n, n * C
        self.K, self.nC = K, nC
        sizes = [K * nC, K, 4, C]                 # alpha padded to 4 so every slice is 16-byte aligned
        self.flat = torch.zeros(sum(sizes), dtype=torch.float32, device=device)
        o = 0
        self.d_phi = self.flat[o:o + K * nC].view(K, nC); o += K * nC
        self.d_bias = self.flat[o:o + K]; o += K
        self.d_alpha = self.flat[o:o + 3]; o += 4
        self.d_rmsnorm_weight = self.flat[o:o + C]

    def as_grads(self):
        """The dict ``capi.dynamic_bwd(..., grads=...)`` writes into."""
        return {"d_rmsnorm_weight": self.d_rmsnorm_weight, "d_phi": self.d_phi,
                "d_alpha": self.d_alpha, "d_bias": self.d_bias}

    def all_reduce(self, group=None, async_op=False):
        """Sum the bucket over the data-parallel group (no-op without an initialised group)."""
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
            return None
        return dist.all_reduce(self.flat, op=dist.ReduceOp.SUM, group=group, async_op=async_op)

    def to_param_grads(self):
        """Views of the bucket under the layer's parameter names (``MHCLayer`` layout)."""
        n = self.n
        return {
            "rmsnorm_weight": self.d_rmsnorm_weight,
            "phi_pre": self.d_phi[:n], "phi_post": self.d_phi[n:2 * n], "phi_res": self.d_phi[2 * n:],
            "alpha_pre": self.d_alpha[0], "alpha_post": self.d_alpha[1], "alpha_res": self.d_alpha[2],
            "b_pre": self.d_bias[:n], "b_post": self.d_bias[n:2 * n],
            "b_res": self.d_bias[2 * n:].view(n, n),
        }
