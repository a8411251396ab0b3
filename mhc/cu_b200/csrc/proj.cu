// The two contractions against phi whose reduction axis is long:
//   proj   praw[b,k] = sum_m x_flat[b,m] * phi[k,m]   and   sumsq[b] = sum_m x_flat[b,m]^2
//   dphi   dphi[k,m] = sum_b dpr[b,k] * x_flat[b,m]
// This file holds the fp32-FMA versions: they serve fp32 I/O (where 1e-5 parity rules out
// reduced-precision tensor-core inputs) and every shape the bf16 tensor-core kernels do not cover.
//
// Takes over compute_rms + the cuBLASLt projection GEMM (src/csrc/kernels/fused_rmsnorm_matmul.cuh:
// 15-153, src/python/bindings.cu:21-111,426-443) and the eager d_phi GEMMs
// (src/python/mhc/ops.py:330-332) of the reference.
#include "kernels.h"

namespace mhc {

namespace {

constexpr int kProjTokens = 8;  // tokens per block
constexpr int kProjRows = 8;    // phi rows per block
constexpr int kProjThreads = 256;

template <typename T, int V>
__global__ void __launch_bounds__(kProjThreads)
proj_kernel(float* __restrict__ praw, float* __restrict__ sumsq, const T* __restrict__ x,
            const T* __restrict__ phi, int64_t B, int K, int64_t nC) {
    constexpr int NV = kProjTokens * kProjRows + kProjTokens;
    __shared__ float red[NV * 32];
    const int64_t b0 = (int64_t)blockIdx.x * kProjTokens;
    const int k0 = blockIdx.y * kProjRows;
    const int64_t nvec = nC / V;

    float acc[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[i] = 0.f;

    for (int64_t v = threadIdx.x; v < nvec; v += kProjThreads) {
        float xv[kProjTokens][V];
#pragma unroll
        for (int t = 0; t < kProjTokens; ++t) {
            if (b0 + t < B) {
                load_vec<V>(x + (b0 + t) * nC + v * V, xv[t]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) xv[t][e] = 0.f;
            }
        }
#pragma unroll
        for (int r = 0; r < kProjRows; ++r) {
            if (k0 + r < K) {
                float pv[V];
                load_vec<V>(phi + (int64_t)(k0 + r) * nC + v * V, pv);
#pragma unroll
                for (int t = 0; t < kProjTokens; ++t) {
#pragma unroll
                    for (int e = 0; e < V; ++e)
                        acc[t * kProjRows + r] = fmaf(xv[t][e], pv[e], acc[t * kProjRows + r]);
                }
            }
        }
        if (blockIdx.y == 0) {
#pragma unroll
            for (int t = 0; t < kProjTokens; ++t) {
#pragma unroll
                for (int e = 0; e < V; ++e)
                    acc[kProjTokens * kProjRows + t] =
                        fmaf(xv[t][e], xv[t][e], acc[kProjTokens * kProjRows + t]);
            }
        }
    }
    block_sum<NV>(acc, red);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int t = 0; t < kProjTokens; ++t) {
            if (b0 + t < B) {
#pragma unroll
                for (int r = 0; r < kProjRows; ++r)
                    if (k0 + r < K) praw[(b0 + t) * K + k0 + r] = acc[t * kProjRows + r];
                if (blockIdx.y == 0) sumsq[b0 + t] = acc[kProjTokens * kProjRows + t];
            }
        }
    }
}

// Block = 32 column vectors x 8 token lanes; it owns kDphiRows rows of dphi for its columns and
// walks all tokens, so every element of dphi is written exactly once, in a fixed order.
constexpr int kDphiRows = 8;
constexpr int kDphiTY = 8;

template <typename T, int V>
__global__ void __launch_bounds__(256)
dphi_kernel(float* __restrict__ dphi, const T* __restrict__ x, const float* __restrict__ dpr,
            int64_t B, int K, int64_t nC) {
    __shared__ float sm[kDphiTY][32][V];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t nvec = nC / V;
    const int64_t v = (int64_t)blockIdx.x * 32 + tx;
    const bool colact = v < nvec;
    const int k0 = blockIdx.y * kDphiRows;

    float acc[kDphiRows][V];
#pragma unroll
    for (int r = 0; r < kDphiRows; ++r)
#pragma unroll
        for (int e = 0; e < V; ++e) acc[r][e] = 0.f;

    if (colact) {
#pragma unroll 4
        for (int64_t b = ty; b < B; b += kDphiTY) {
            float xv[V];
            load_vec<V>(x + b * nC + v * V, xv);
            const float* dp = dpr + b * K + k0;
#pragma unroll
            for (int r = 0; r < kDphiRows; ++r) {
                if (k0 + r < K) {
                    const float dk = dp[r];
#pragma unroll
                    for (int e = 0; e < V; ++e) acc[r][e] = fmaf(dk, xv[e], acc[r][e]);
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < kDphiRows; ++r) {
        __syncthreads();
#pragma unroll
        for (int e = 0; e < V; ++e) sm[ty][tx][e] = acc[r][e];
        __syncthreads();
        if (ty == 0 && colact && k0 + r < K) {
            float o[V];
#pragma unroll
            for (int e = 0; e < V; ++e) {
                float t = 0.f;
#pragma unroll
                for (int l = 0; l < kDphiTY; ++l) t += sm[l][tx][e];
                o[e] = t;
            }
            store_vec<V>(dphi + (int64_t)(k0 + r) * nC + v * V, o);
        }
    }
}

}  // namespace

template <typename T>
cudaError_t launch_proj(float* praw, float* sumsq, const T* x, const T* phi, Dims d,
                        cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    constexpr int VW = VecWidth<T>::value;
    const int K = d.K();
    const dim3 grid((unsigned)((d.B + kProjTokens - 1) / kProjTokens),
                    (unsigned)((K + kProjRows - 1) / kProjRows));
    if (d.nC() % VW == 0 && d.C % VW == 0)
        proj_kernel<T, VW><<<grid, kProjThreads, 0, s>>>(praw, sumsq, x, phi, d.B, K, d.nC());
    else
        proj_kernel<T, 1><<<grid, kProjThreads, 0, s>>>(praw, sumsq, x, phi, d.B, K, d.nC());
    return launched();
}

template <typename T>
cudaError_t launch_dphi(float* dphi, const T* x, const float* dpr, Dims d, cudaStream_t s) {
    constexpr int VW = VecWidth<T>::value;
    const int K = d.K();
    const bool vec = (d.C % VW == 0) && (d.nC() % 4 == 0);
    const int64_t nvec = vec ? d.nC() / VW : d.nC();
    const dim3 block(32, kDphiTY);
    const dim3 grid((unsigned)((nvec + 31) / 32), (unsigned)((K + kDphiRows - 1) / kDphiRows));
    if (vec)
        dphi_kernel<T, VW><<<grid, block, 0, s>>>(dphi, x, dpr, d.B, K, d.nC());
    else
        dphi_kernel<T, 1><<<grid, block, 0, s>>>(dphi, x, dpr, d.B, K, d.nC());
    return launched();
}

template cudaError_t launch_proj<float>(float*, float*, const float*, const float*, Dims,
                                        cudaStream_t);
template cudaError_t launch_proj<bf16>(float*, float*, const bf16*, const bf16*, Dims,
                                       cudaStream_t);
template cudaError_t launch_dphi<float>(float*, const float*, const float*, Dims, cudaStream_t);
template cudaError_t launch_dphi<bf16>(float*, const bf16*, const float*, Dims, cudaStream_t);

}  // namespace mhc
