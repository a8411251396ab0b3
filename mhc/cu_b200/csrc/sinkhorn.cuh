// Sinkhorn-Knopp on one n x n matrix held by a group of G consecutive lanes (G a power of two,
// n <= G <= 32): lane r of the group keeps row r in registers.  Row sums are thread-local, column
// sums are G-wide xor-butterflies.  Several groups share a warp, so small n packs 32/G matrices
// per warp.  A is float or double.
//
// Each normalisation step divides by (sum + eps) — the semantics of the naive layer
// (src/python/tests/test_layer.py:38-41 of the reference) — not the reference kernels'
// "divide by sum only if sum > eps" (src/csrc/kernels/sinkhorn_knopp.cuh:854-857).
#pragma once

#include "common.cuh"

namespace mhc {

template <int G, typename A>
__device__ __forceinline__ A group_sum(A v) {
#pragma unroll
    for (int o = G / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int G, typename A>
__device__ __forceinline__ A group_get(A v, int lane_in_group) {
    return __shfl_sync(0xffffffffu, v, lane_in_group, G);
}

template <typename A>
__device__ __forceinline__ A sk_exp(A v);
template <>
__device__ __forceinline__ float sk_exp<float>(float v) { return expf(v); }
template <>
__device__ __forceinline__ double sk_exp<double>(double v) { return exp(v); }

template <typename A>
__device__ __forceinline__ A sk_sigmoid(A t) { return A(1) / (A(1) + sk_exp<A>(-t)); }

// Forward.  m[] holds this lane's row on entry (zeros for j >= n and for lanes with row >= n)
// and the normalised row on return.  With STORE, den[2t] receives the (row sum + eps) of step t
// for this lane's row and den[2t+1] the (column sum + eps) of column `row`.
// Must be called by all 32 lanes of the warp.
template <int G, typename A, bool STORE>
__device__ __forceinline__ void sk_forward(A (&m)[G], int n, int row, int iters, A eps, A* den) {
    const bool act = row < n;
    for (int t = 0; t < iters; ++t) {
        A rs = A(0);
#pragma unroll
        for (int j = 0; j < G; ++j)
            if (j < n) rs += m[j];
        const A rd = rs + eps;
        const A rinv = A(1) / rd;
        if (act) {
#pragma unroll
            for (int j = 0; j < G; ++j)
                if (j < n) m[j] *= rinv;
        }
        A mycd = A(1);
#pragma unroll
        for (int j = 0; j < G; ++j) {
            if (j < n) {
                const A cd = group_sum<G, A>(m[j]) + eps;
                if (act) m[j] *= A(1) / cd;
                if (j == row) mycd = cd;
            }
        }
        if (STORE && act) {
            den[2 * t] = rd;
            den[2 * t + 1] = mycd;
        }
    }
}

// Backward through all 2*iters steps.  On entry d[] is dL/dM for this lane's row and y[] the
// forward's result; on return d[] is dL/dE and y[] the rebuilt input E (up to rounding).
// For y = x / (s + eps): dx = (dy - sum_axis(dy*y)) / (s + eps) and x = y * (s + eps).
template <int G, typename A>
__device__ __forceinline__ void sk_backward(A (&d)[G], A (&y)[G], int n, int row, int iters,
                                            const A* den) {
    const bool act = row < n;
    for (int t = iters - 1; t >= 0; --t) {
        const A mycd = act ? den[2 * t + 1] : A(1);
#pragma unroll
        for (int j = 0; j < G; ++j) {
            if (j < n) {
                const A cd = group_get<G, A>(mycd, j);
                const A tc = group_sum<G, A>(d[j] * y[j]);
                if (act) {
                    d[j] = (d[j] - tc) / cd;
                    y[j] *= cd;
                }
            }
        }
        const A rd = act ? den[2 * t] : A(1);
        A tr = A(0);
#pragma unroll
        for (int j = 0; j < G; ++j)
            if (j < n) tr += d[j] * y[j];
        if (act) {
            const A rinv = A(1) / rd;
#pragma unroll
            for (int j = 0; j < G; ++j) {
                if (j < n) {
                    d[j] = (d[j] - tr) * rinv;
                    y[j] *= rd;
                }
            }
        }
    }
}

}  // namespace mhc
