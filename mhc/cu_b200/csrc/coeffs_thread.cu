// Per-token backward algebra with ONE THREAD PER TOKEN (n <= 8): the token's n x n matrices live
// in that thread's registers, so the 2*iters Sinkhorn steps need no shuffles and the n rows
// (columns) of a step are independent instruction chains.  A warp handles 32 tokens; its
// token-summed outputs (d_bias, d_alpha terms) are added in shared memory in token order and
// leave the block as one partial row, so the final sums are bit-reproducible.
//
// Same inputs / outputs as coeffs_dyn_bwd_kernel in coeffs.cu (which remains for n > 8).
#include "kernels.h"
#include "sinkhorn.cuh"
#include "coeffs_lanes.cuh"

namespace mhc {

namespace {

constexpr int kTokThreads = 32;

template <int MAXN, typename A>
__global__ void __launch_bounds__(kTokThreads)
coeffs_dyn_bwd_thread_kernel(float* __restrict__ dpr, float* __restrict__ qq,
                             float* __restrict__ partials, const float* __restrict__ dH,
                             const float* __restrict__ H_pre, const float* __restrict__ H_post,
                             const float* __restrict__ proj, const float* __restrict__ rms_h,
                             const float* __restrict__ alpha, const float* __restrict__ bias,
                             A* __restrict__ den_ws, int64_t B, int n, int64_t nC, int iters,
                             float eps, MmaBwdOut mo, int den_in_smem) {
    extern __shared__ __align__(16) float sm[];   // [kTokThreads][K+3], then the denominators
    const int K = 2 * n + n * n;
    const int KP = K + 3;
    const int K8P = (K + 7) / 8 * 8;
    const int64_t Bp = (B + 15) / 16 * 16;
    const int64_t tok = (int64_t)blockIdx.x * kTokThreads + threadIdx.x;
    const bool act = tok < B;
    float* smt = sm + threadIdx.x * KP;
    for (int k = 0; k < KP; ++k) smt[k] = 0.f;

    if (act) {
        const float* pj = proj + tok * K;
        const float* dh = dH + tok * K;
        const A a0 = A(alpha[0]), a1 = A(alpha[1]), a2 = A(alpha[2]);
        A y[MAXN][MAXN], d[MAXN][MAXN];
#pragma unroll
        for (int i = 0; i < MAXN; ++i)
#pragma unroll
            for (int j = 0; j < MAXN; ++j) {
                const bool in = (i < n) && (j < n);
                const int k = 2 * n + i * n + j;
                y[i][j] = in ? sk_exp<A>(a2 * A(pj[k]) + A(bias[k])) : A(0);
                d[i][j] = in ? A(dh[k]) : A(0);
            }
        // Sinkhorn denominators of the forward sweep: in shared memory (one column per thread,
        // conflict-free) when they fit, else in the global workspace
        A* den;
        int ds;
        if (den_in_smem) {
            const int off = (kTokThreads * KP * (int)sizeof(float) + 15) / 16 * 16;
            den = reinterpret_cast<A*>(reinterpret_cast<unsigned char*>(sm) + off) + threadIdx.x;
            ds = kTokThreads;
        } else {
            den = den_ws + tok * 2 * (int64_t)iters * MAXN;
            ds = 1;
        }
        sk_forward_thread<MAXN, A, true>(y, n, iters, A(eps), den, ds);
        sk_backward_thread<MAXN, A>(d, y, n, iters, den, ds);

        const A r = A(rms_h[tok]);
        const A rinv = A(1) / r;
        float* dpo = dpr + tok * K;
        A qacc = A(0), dal0 = A(0), dal1 = A(0), dal2 = A(0);
        const int RS = (n * n + 2 * n + 3 + 3) / 4 * 4;
        float* rc = (mo.rec != nullptr) ? mo.rec + tok * RS : nullptr;
        for (int i = 0; i < n; ++i) {
            const A hp = A(H_pre[tok * n + i]), hq = A(H_post[tok * n + i]);
            const A pp = A(pj[i]), pq = A(pj[n + i]);
            const A dtp = A(dh[i]) * hp * (A(1) - hp);
            const A dtq = A(dh[n + i]) * hq * (A(1) - hq * A(0.5));
            const A vp = a0 * dtp * rinv, vq = a1 * dtq * rinv;
            dpo[i] = (float)vp;
            dpo[n + i] = (float)vq;
            smt[i] = (float)dtp;
            smt[n + i] = (float)dtq;
            qacc += vp * pp + vq * pq;
            dal0 += dtp * pp;
            dal1 += dtq * pq;
            if (rc != nullptr) {
                rc[n * n + i] = (float)hp;
                rc[n * n + n + i] = (float)hq;
                mo.dprb[tok * K8P + i] = __float2bfloat16_rn((float)vp);
                mo.dprb[tok * K8P + n + i] = __float2bfloat16_rn((float)vq);
                mo.dprT[(int64_t)i * Bp + tok] = __float2bfloat16_rn((float)vp);
                mo.dprT[(int64_t)(n + i) * Bp + tok] = __float2bfloat16_rn((float)vq);
            }
        }
#pragma unroll
        for (int i = 0; i < MAXN; ++i)
#pragma unroll
            for (int j = 0; j < MAXN; ++j) {
                if (i < n && j < n) {
                    const int k = 2 * n + i * n + j;
                    const A dtr = d[i][j] * y[i][j];   // dE * E (E rebuilt by the reverse sweep)
                    const A pv = A(pj[k]);
                    const A v = a2 * dtr * rinv;
                    dpo[k] = (float)v;
                    smt[k] = (float)dtr;
                    qacc += v * pv;
                    dal2 += dtr * pv;
                    if (rc != nullptr) {
                        rc[j * n + i] = mo.M[tok * n * n + i * n + j];   // MT[j][i] = M[i][j]
                        mo.dprb[tok * K8P + k] = __float2bfloat16_rn((float)v);
                        mo.dprT[(int64_t)k * Bp + tok] = __float2bfloat16_rn((float)v);
                    }
                }
            }
        const float qv = (float)(qacc / (A(nC) * r));
        qq[tok] = qv;
        smt[K] = (float)dal0;
        smt[K + 1] = (float)dal1;
        smt[K + 2] = (float)dal2;
        if (rc != nullptr) {
            rc[n * n + 2 * n] = 1.f / mo.rms[tok];
            rc[n * n + 2 * n + 1] = mo.c2[tok];
            rc[n * n + 2 * n + 2] = qv;
            for (int k = K; k < K8P; ++k) {
                mo.dprb[tok * K8P + k] = __float2bfloat16_rn(0.f);
                mo.dprT[(int64_t)k * Bp + tok] = __float2bfloat16_rn(0.f);
            }
        }
    } else if (mo.rec != nullptr && tok < Bp) {
        // padding tokens of the k-major bf16 copy
        for (int k = 0; k < K8P; ++k) mo.dprT[(int64_t)k * Bp + tok] = __float2bfloat16_rn(0.f);
    }
    __syncthreads();
    for (int k = threadIdx.x; k < KP; k += kTokThreads) {
        float t = 0.f;
        for (int g = 0; g < kTokThreads; ++g) t += sm[g * KP + k];
        partials[(int64_t)blockIdx.x * KP + k] = t;
    }
}

}  // namespace

int coeffs_thread_blocks(Dims d) {
    const int64_t Bp = (d.B + 15) / 16 * 16;
    return (int)((Bp + kTokThreads - 1) / kTokThreads);
}

// floats / doubles of Sinkhorn denominators per token
int coeffs_thread_den_per_token(Dims d, int iters) { return 2 * iters * (d.n <= 4 ? 4 : 8); }

cudaError_t launch_coeffs_dyn_bwd_thread(float* dpr, float* qq, float* partials, const float* dH,
                                         const float* H_pre, const float* H_post,
                                         const float* proj, const float* rms_h,
                                         const float* alpha, const float* bias, void* den_ws,
                                         Dims d, int iters, float eps, bool use_double,
                                         MmaBwdOut mo, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (d.n > 8) return cudaErrorNotSupported;
    const unsigned grid = (unsigned)coeffs_thread_blocks(d);
    const size_t part = ((size_t)kTokThreads * (d.K() + 3) * sizeof(float) + 15) / 16 * 16;
    const size_t den_bytes = (size_t)kTokThreads * 2 * iters * (d.n <= 4 ? 4 : 8) *
                             (use_double ? sizeof(double) : sizeof(float));
    const int den_in_smem = (part + den_bytes <= 48 * 1024) ? 1 : 0;
    const size_t smem = part + (den_in_smem ? den_bytes : 0);
#define MHC_CT(MAXN_, A_)                                                                          \
    coeffs_dyn_bwd_thread_kernel<MAXN_, A_><<<grid, kTokThreads, smem, s>>>(                       \
        dpr, qq, partials, dH, H_pre, H_post, proj, rms_h, alpha, bias, (A_*)den_ws, d.B, d.n,     \
        d.nC(), iters, eps, mo, den_in_smem)
    if (d.n <= 4) {
        if (use_double) MHC_CT(4, double); else MHC_CT(4, float);
    } else {
        if (use_double) MHC_CT(8, double); else MHC_CT(8, float);
    }
#undef MHC_CT
    return launched();
}

}  // namespace mhc

// ------------------------------------------------------------------------------------------------
// n <= 4, float: SIXTEEN LANES PER TOKEN (one per matrix element) and the Sinkhorn denominators
// saved by the forward, so only the reverse sweep runs here and each of its 2*iters steps is a
// two-shuffle sum plus three arithmetic instructions.  Block = 256 threads = 16 tokens.
namespace mhc {

namespace {

constexpr int kLaneTokens = 16;

__global__ void __launch_bounds__(256)
coeffs_dyn_bwd_lanes_kernel(float* __restrict__ dpr, float* __restrict__ qq,
                            float* __restrict__ partials, const float* __restrict__ dH,
                            const float* __restrict__ H_pre, const float* __restrict__ H_post,
                            const float* __restrict__ M, const float* __restrict__ proj,
                            const float* __restrict__ rms_h, const float* __restrict__ alpha,
                            const float* __restrict__ bias, const float* __restrict__ sk_den,
                            int64_t B, int n, int64_t nC, int iters, MmaBwdOut mo) {
    extern __shared__ __align__(16) float sm[];   // [16][K+3] token sums, then [16][2*iters*4] den
    const int K = 2 * n + n * n, KP = K + 3;
    const int tl = threadIdx.x >> 4, e = threadIdx.x & 15;   // token slot, element
    const int i = e >> 2, j = e & 3;
    const int64_t tok = (int64_t)blockIdx.x * kLaneTokens + tl;
    const bool act = tok < B;
    const bool elem = act && i < n && j < n;
    const int dpt = 2 * iters * 4;                            // denominators per token
    float* part = sm;
    float* den = sm + kLaneTokens * KP;
    for (int k = threadIdx.x; k < kLaneTokens * KP; k += 256) part[k] = 0.f;
    {   // coalesced copy of the block's denominators
        const int64_t base = (int64_t)blockIdx.x * kLaneTokens * dpt;
        const int64_t lim = B * dpt;
        for (int k = threadIdx.x; k < kLaneTokens * dpt; k += 256)
            den[k] = (base + k < lim) ? sk_den[base + k] : 1.f;
    }
    __syncthreads();

    LaneIn in{0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (elem) {
        const int k_res = 2 * n + i * n + j;
        in.m = M[tok * n * n + i * n + j];
        in.dres = dH[tok * K + k_res];
        in.p_res = proj[tok * K + k_res];
    }
    if (act && e < 2 * n) {
        in.h = (e >= n) ? H_post[tok * n + (e - n)] : H_pre[tok * n + e];
        in.dh = dH[tok * K + e];
        in.p_e = proj[tok * K + e];
    }
    const float r = act ? rms_h[tok] : 1.f;
    const float c1 = (act && mo.rec != nullptr) ? 1.f / mo.rms[tok] : 0.f;
    const float c2v = (act && mo.rec != nullptr) ? mo.c2[tok] : 0.f;
    coeffs_lanes_token(tok, act, e, n, nC, iters, B, in, r, alpha[0], alpha[1], alpha[2], c1, c2v,
                       den + tl * dpt, part + tl * KP, dpr, qq, mo);
    __syncthreads();
    for (int k = threadIdx.x; k < KP; k += 256) {
        float t = 0.f;
        for (int g = 0; g < kLaneTokens; ++g) t += part[g * KP + k];
        partials[(int64_t)blockIdx.x * KP + k] = t;
    }
}

}  // namespace

// The lane kernel needs n <= 4, the forward's denominators, and room for them in shared memory.
bool coeffs_lanes_supported(Dims d, int iters) {
    return d.n <= 4 && (size_t)kLaneTokens * (d.K() + 3 + 2 * iters * 4) * sizeof(float) <= 40 * 1024;
}

int coeffs_lanes_blocks(Dims d) {
    const int64_t Bp = (d.B + 15) / 16 * 16;
    return (int)(Bp / kLaneTokens);
}

cudaError_t launch_coeffs_dyn_bwd_lanes(float* dpr, float* qq, float* partials, const float* dH,
                                        const float* H_pre, const float* H_post, const float* M,
                                        const float* proj, const float* rms_h, const float* alpha,
                                        const float* bias, const float* sk_den, Dims d, int iters,
                                        MmaBwdOut mo, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!coeffs_lanes_supported(d, iters)) return cudaErrorNotSupported;
    const size_t smem = (size_t)kLaneTokens * (d.K() + 3 + 2 * iters * 4) * sizeof(float);
    coeffs_dyn_bwd_lanes_kernel<<<(unsigned)coeffs_lanes_blocks(d), 256, smem, s>>>(
        dpr, qq, partials, dH, H_pre, H_post, M, proj, rms_h, alpha, bias, sk_den, d.B, d.n, d.nC(),
        iters, mo);
    return launched();
}

}  // namespace mhc
