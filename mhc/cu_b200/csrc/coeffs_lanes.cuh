// Backward of one token's coefficients with SIXTEEN LANES PER TOKEN (n <= 4, fp32): lane e holds
// element (i, j) = (e / 4, e % 4) of the Sinkhorn matrix.  With the denominators the forward saved,
// only the reverse sweep runs, and each of its 2 * iters steps is a two-shuffle sum plus three
// arithmetic instructions.  Shared by the stand-alone coefficient kernel and by the epilogue of
// the Gram pass (bwd_gram.cu), which calls it for the two tokens of its block.
//
// Follows the backward of sinkhorn_knopp / the dynamic-H activations in the reference
// (src/csrc/kernels/sinkhorn_knopp.cuh:366-560, src/python/mhc/ops.py:300-349).
#pragma once
#include "kernels.h"
#include "sinkhorn.cuh"

namespace mhc {

// Per-lane inputs of coeffs_lanes_token, fetched by the caller (so that it can fetch them early).
struct LaneIn {
    float m;        // M[i][j]                       (lanes with i, j < n; else 0)
    float dres;     // dL/dM[i][j] = dH[2n + i n + j] (same lanes; else 0)
    float p_res;    // proj[2n + i n + j]
    float h;        // lanes e < n: H_pre[e]; n <= e < 2n: H_post[e - n]
    float dh;       // dH[e] for e < 2n
    float p_e;      // proj[e] for e < 2n
};

// All 32 lanes of the warp call this together (each half-warp one token; `act` false for a token
// slot beyond the batch).  dn: this token's saved denominators [2*iters][4] (shared memory);
// pt: [K+3] floats of shared memory that receive the token's terms of d_bias (K) and d_alpha (3);
// they are NOT written for an inactive slot.  c1 = 1 / rho, c2v = the token's c2, r = rms_h.
__device__ __forceinline__ void coeffs_lanes_token(int64_t tok, bool act, int e, int n, int64_t nC,
                                                   int iters, int64_t B, const LaneIn& in, float r,
                                                   float al0, float al1, float al2, float c1,
                                                   float c2v, const float* dn, float* pt, float* dpr,
                                                   float* qq, const MmaBwdOut& mo) {
    const int K = 2 * n + n * n, K8P = (K + 7) / 8 * 8;
    const int64_t Bp = (B + 15) / 16 * 16;
    const int i = e >> 2, j = e & 3;
    const bool elem = act && i < n && j < n;
    const int k_res = 2 * n + i * n + j;
    float y = elem ? in.m : 0.f;
    float d = elem ? in.dres : 0.f;
    for (int t = iters - 1; t >= 0; --t) {
        // lanes outside the n x n matrix carry zeros; their slots of the saved denominators are
        // never written, so they take 1 instead of reading them
        const float cd = elem ? dn[(2 * t + 1) * 4 + j] : 1.f;
        float tc = d * y;
        tc += __shfl_xor_sync(0xffffffffu, tc, 4);
        tc += __shfl_xor_sync(0xffffffffu, tc, 8);
        d = (d - tc) * sk_rcp<float>(cd);
        y *= cd;
        const float rd = elem ? dn[(2 * t) * 4 + i] : 1.f;
        float tr = d * y;
        tr += __shfl_xor_sync(0xffffffffu, tr, 1);
        tr += __shfl_xor_sync(0xffffffffu, tr, 2);
        d = (d - tr) * sk_rcp<float>(rd);
        y *= rd;
    }
    // y is now E = exp(t_res) (rebuilt), d = dL/dE
    const float rinv = 1.f / r;
    const int RS = (n * n + 2 * n + 3 + 3) / 4 * 4;
    float* rc = (mo.rec != nullptr && act) ? mo.rec + tok * RS : nullptr;
    float qacc = 0.f, dal0 = 0.f, dal1 = 0.f, dal2 = 0.f;
    if (elem) {
        const float dtr = d * y;
        const float v = al2 * dtr * rinv;
        dpr[tok * K + k_res] = v;
        pt[k_res] = dtr;
        qacc = v * in.p_res;
        dal2 = dtr * in.p_res;
        if (rc != nullptr) {
            rc[j * n + i] = in.m;   // MT[j][i] = M[i][j]
            mo.dprb[tok * K8P + k_res] = __float2bfloat16_rn(v);
            mo.dprT[(int64_t)k_res * Bp + tok] = __float2bfloat16_rn(v);
        }
    }
    if (act && e < 2 * n) {   // lanes 0..n-1: the pre entries, n..2n-1: the post entries
        const bool post = e >= n;
        const float h = in.h;
        const float dt = post ? in.dh * h * (1.f - 0.5f * h) : in.dh * h * (1.f - h);
        const float v = (post ? al1 : al0) * dt * rinv;
        dpr[tok * K + e] = v;
        pt[e] = dt;
        qacc += v * in.p_e;
        if (post) dal1 = dt * in.p_e; else dal0 = dt * in.p_e;
        if (rc != nullptr) {
            rc[n * n + e] = h;   // H_pre at n*n + i, H_post at n*n + n + i
            mo.dprb[tok * K8P + e] = __float2bfloat16_rn(v);
            mo.dprT[(int64_t)e * Bp + tok] = __float2bfloat16_rn(v);
        }
    }
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        qacc += __shfl_xor_sync(0xffffffffu, qacc, o);
        dal0 += __shfl_xor_sync(0xffffffffu, dal0, o);
        dal1 += __shfl_xor_sync(0xffffffffu, dal1, o);
        dal2 += __shfl_xor_sync(0xffffffffu, dal2, o);
    }
    if (act && e == 0) {
        const float qv = qacc / ((float)nC * r);
        qq[tok] = qv;
        pt[K] = dal0;
        pt[K + 1] = dal1;
        pt[K + 2] = dal2;
        if (rc != nullptr) {
            rc[n * n + 2 * n] = c1;
            rc[n * n + 2 * n + 1] = c2v;
            rc[n * n + 2 * n + 2] = qv;
        }
    }
    if (mo.rec != nullptr && tok < Bp) {
        // zero padding of the bf16 copies: rows K..K8P-1, and all rows of the tokens B..Bp-1
        for (int k = e; k < K8P; k += 16) {
            if (!act) {
                mo.dprT[(int64_t)k * Bp + tok] = __float2bfloat16_rn(0.f);
            } else if (k >= K) {
                mo.dprb[tok * K8P + k] = __float2bfloat16_rn(0.f);
                mo.dprT[(int64_t)k * Bp + tok] = __float2bfloat16_rn(0.f);
            }
        }
    }
}

}  // namespace mhc
