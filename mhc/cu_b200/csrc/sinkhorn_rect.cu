// Stand-alone Sinkhorn-Knopp on ONE rectangular matrix [M, N], M, N <= 128 (the shape range of the
// reference's single-matrix op), forward and exact backward.
//
//   out = inp;  repeat iters times:  out[i,:] /= (sum_j out[i,j] + eps);  out[:,j] /= (sum_i out[i,j] + eps)
//
// One block of 1024 threads, the matrix in shared memory.  Row sums: one warp per row (lanes
// stride over the columns); column sums: eight threads per column, combined by shuffles.  The
// backward first repeats the forward sweep keeping every denominator (2 * iters * 128 floats of
// workspace), then walks the steps in reverse with  d <- (d - <d, y>_line) / den,  y <- y * den,
// the same recurrence the batched kernels use; the line sums are accumulated in fp64.
//
// Takes over sinkhorn_knopp_forward / sinkhorn_knopp_backward of the reference for 2-D inputs
// (src/python/bindings.cu:115-132, src/csrc/kernels/sinkhorn_knopp.cuh:423-459,586-825).  The
// reference's backward accepts square matrices only; this one takes any M, N <= 128.
#include "kernels.h"

namespace mhc {

namespace {

constexpr int kRectMax = 128;
constexpr int kRectThreads = 1024;

// One Sinkhorn step on the shared-memory matrix m [M][N] (pitch N).  rden / cden (optional) receive
// the row / column denominators of this step.
__device__ __forceinline__ void rect_step(float* m, int M, int N, float eps, float* rden, float* cden,
                                          float* colinv) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = warp; i < M; i += kRectThreads / 32) {
        float s = 0.f;
        for (int j = lane; j < N; j += 32) s += m[i * N + j];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        const float d = s + eps;
        const float inv = 1.f / d;
        for (int j = lane; j < N; j += 32) m[i * N + j] *= inv;
        if (rden != nullptr && lane == 0) rden[i] = d;
    }
    __syncthreads();
    {   // eight threads per column: thread (j, part) adds rows part, part + 8, ...
        const int j = tid >> 3, part = tid & 7;
        float s = 0.f;
        if (j < N)
            for (int i = part; i < M; i += 8) s += m[i * N + j];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (j < N && part == 0) {
            const float d = s + eps;
            colinv[j] = 1.f / d;
            if (cden != nullptr) cden[j] = d;
        }
    }
    __syncthreads();
    for (int k = tid; k < M * N; k += kRectThreads) m[k] *= colinv[k % N];
    __syncthreads();
}

__global__ void __launch_bounds__(kRectThreads)
sinkhorn_rect_fwd_kernel(float* __restrict__ out, const float* __restrict__ inp, int M, int N,
                         int iters, float eps) {
    extern __shared__ __align__(16) float sm[];   // [M*N] matrix, [128] column scale
    float* m = sm;
    float* colinv = sm + M * N;
    for (int k = threadIdx.x; k < M * N; k += kRectThreads) m[k] = inp[k];
    __syncthreads();
    for (int t = 0; t < iters; ++t) rect_step(m, M, N, eps, nullptr, nullptr, colinv);
    for (int k = threadIdx.x; k < M * N; k += kRectThreads) out[k] = m[k];
}

// den: [2*iters][128] floats of global workspace (row denominators of step t at (2t)*128 + i,
// column denominators at (2t+1)*128 + j)
__global__ void __launch_bounds__(kRectThreads)
sinkhorn_rect_bwd_kernel(float* __restrict__ d_inp, const float* __restrict__ grad,
                         const float* __restrict__ inp, float* __restrict__ den, int M, int N,
                         int iters, float eps) {
    extern __shared__ __align__(16) float sm[];   // y [M*N], d [M*N], line [128]
    float* y = sm;
    float* d = sm + M * N;
    float* line = d + M * N;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int k = tid; k < M * N; k += kRectThreads) {
        y[k] = inp[k];
        d[k] = grad[k];
    }
    __syncthreads();
    for (int t = 0; t < iters; ++t)
        rect_step(y, M, N, eps, den + (2 * t) * kRectMax, den + (2 * t + 1) * kRectMax, line);
    __threadfence_block();
    __syncthreads();
    for (int t = iters - 1; t >= 0; --t) {
        // column step backwards:  d[i,j] <- (d[i,j] - sum_i d y) / cd[j],  y <- y * cd[j]
        {
            const int j = tid >> 3, part = tid & 7;
            double s = 0.0;
            if (j < N)
                for (int i = part; i < M; i += 8) s += (double)d[i * N + j] * (double)y[i * N + j];
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            if (j < N && part == 0) line[j] = (float)s;
        }
        __syncthreads();
        {
            const float* cd = den + (2 * t + 1) * kRectMax;
            for (int k = tid; k < M * N; k += kRectThreads) {
                const int j = k % N;
                const float c = cd[j];
                d[k] = (d[k] - line[j]) / c;
                y[k] *= c;
            }
        }
        __syncthreads();
        // row step backwards
        {
            const float* rd = den + (2 * t) * kRectMax;
            for (int i = warp; i < M; i += kRectThreads / 32) {
                double s = 0.0;
                for (int j = lane; j < N; j += 32) s += (double)d[i * N + j] * (double)y[i * N + j];
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
                const float sf = (float)s, r = rd[i];
                for (int j = lane; j < N; j += 32) {
                    d[i * N + j] = (d[i * N + j] - sf) / r;
                    y[i * N + j] *= r;
                }
            }
        }
        __syncthreads();
    }
    for (int k = tid; k < M * N; k += kRectThreads) d_inp[k] = d[k];
}

}  // namespace

size_t sinkhorn_rect_bwd_ws(int iters) { return (size_t)2 * iters * kRectMax * sizeof(float); }

cudaError_t launch_sinkhorn_rect_fwd(float* out, const float* inp, int M, int N, int iters,
                                     float eps, cudaStream_t s) {
    if (M < 1 || N < 1 || M > kRectMax || N > kRectMax) return cudaErrorNotSupported;
    const size_t smem = ((size_t)M * N + kRectMax) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(sinkhorn_rect_fwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    sinkhorn_rect_fwd_kernel<<<1, kRectThreads, smem, s>>>(out, inp, M, N, iters, eps);
    return launched();
}

cudaError_t launch_sinkhorn_rect_bwd(float* d_inp, const float* grad, const float* inp, void* ws,
                                     int M, int N, int iters, float eps, cudaStream_t s) {
    if (M < 1 || N < 1 || M > kRectMax || N > kRectMax) return cudaErrorNotSupported;
    const size_t smem = ((size_t)2 * M * N + kRectMax) * sizeof(float);
    cudaError_t e = cudaFuncSetAttribute(sinkhorn_rect_bwd_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    sinkhorn_rect_bwd_kernel<<<1, kRectThreads, smem, s>>>(d_inp, grad, inp, static_cast<float*>(ws),
                                                          M, N, iters, eps);
    return launched();
}

}  // namespace mhc
