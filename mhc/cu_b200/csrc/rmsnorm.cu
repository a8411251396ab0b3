// Stand-alone RMSNorm over bf16 [B, C] rows with a bf16 weight, forward and backward.
// Takes over rmsnorm_forward_with_rms / rmsnorm_backward (src/csrc/kernels/rmsnorm.cuh:13-306)
// of the reference; d_weight is summed in a fixed order instead of per-element atomicAdd
// (rmsnorm.cuh:293).
#include "kernels.h"

namespace mhc {

namespace {

constexpr int kRmsRowsPerBlock = 64;  // rows per block of the d_weight pass

template <int V>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(bf16* __restrict__ out, float* __restrict__ rms, const bf16* __restrict__ inp,
                   const bf16* __restrict__ w, int64_t C, float eps) {
    __shared__ float red[32];
    __shared__ float inv_s;
    const int64_t b = blockIdx.x;
    const int64_t nvec = C / V;
    const bf16* xb = inp + b * C;
    float ss = 0.f;
    for (int64_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float xv[V];
        load_vec<V>(xb + v * V, xv);
#pragma unroll
        for (int e = 0; e < V; ++e) ss = fmaf(xv[e], xv[e], ss);
    }
    float tot[1] = {ss};
    block_sum<1>(tot, red);
    if (threadIdx.x == 0) {
        const float r = sqrtf(tot[0] / (float)C + eps);
        rms[b] = r;
        inv_s = 1.f / r;
    }
    __syncthreads();
    const float ri = inv_s;
    for (int64_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float xv[V], wv[V], o[V];
        load_vec<V>(xb + v * V, xv);
        load_weight<V>(w, v * V, wv);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = xv[e] * ri * wv[e];
        store_vec<V>(out + b * C + v * V, o);
    }
}

// d_inp = g*w/r - x * <g*w, x> / (C r^3)
template <int V>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dx_kernel(bf16* __restrict__ d_inp, const bf16* __restrict__ grad,
                      const bf16* __restrict__ inp, const bf16* __restrict__ w,
                      const float* __restrict__ rms, int64_t C) {
    __shared__ float red[32];
    __shared__ float corr_s;
    const int64_t b = blockIdx.x;
    const int64_t nvec = C / V;
    const bf16* xb = inp + b * C;
    const bf16* gb = grad + b * C;
    float dot = 0.f;
    for (int64_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float xv[V], gv[V], wv[V];
        load_vec<V>(xb + v * V, xv);
        load_vec<V>(gb + v * V, gv);
        load_weight<V>(w, v * V, wv);
#pragma unroll
        for (int e = 0; e < V; ++e) dot = fmaf(gv[e] * wv[e], xv[e], dot);
    }
    float tot[1] = {dot};
    block_sum<1>(tot, red);
    const float ri = 1.f / rms[b];
    if (threadIdx.x == 0) corr_s = tot[0] * ri * ri * ri / (float)C;
    __syncthreads();
    const float corr = corr_s;
    for (int64_t v = threadIdx.x; v < nvec; v += blockDim.x) {
        float xv[V], gv[V], wv[V], o[V];
        load_vec<V>(xb + v * V, xv);
        load_vec<V>(gb + v * V, gv);
        load_weight<V>(w, v * V, wv);
#pragma unroll
        for (int e = 0; e < V; ++e) o[e] = gv[e] * wv[e] * ri - xv[e] * corr;
        store_vec<V>(d_inp + b * C + v * V, o);
    }
}

// dw_part[block_y][c] = sum over the block's rows of g[b,c] * x[b,c] / r[b]
template <int V>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_dw_kernel(float* __restrict__ dw_part, const bf16* __restrict__ grad,
                      const bf16* __restrict__ inp, const float* __restrict__ rms, int64_t B,
                      int64_t C) {
    __shared__ float sm[8][32][V];
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int64_t nvec = C / V;
    const int64_t v = (int64_t)blockIdx.x * 32 + tx;
    const bool colact = v < nvec;
    const int64_t b0 = (int64_t)blockIdx.y * kRmsRowsPerBlock;
    const int64_t b1 = (b0 + kRmsRowsPerBlock < B) ? b0 + kRmsRowsPerBlock : B;
    float acc[V];
#pragma unroll
    for (int e = 0; e < V; ++e) acc[e] = 0.f;
    if (colact) {
        for (int64_t b = b0 + ty; b < b1; b += 8) {
            float xv[V], gv[V];
            load_vec<V>(inp + b * C + v * V, xv);
            load_vec<V>(grad + b * C + v * V, gv);
            const float ri = 1.f / rms[b];
#pragma unroll
            for (int e = 0; e < V; ++e) acc[e] = fmaf(gv[e] * ri, xv[e], acc[e]);
        }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) sm[ty][tx][e] = acc[e];
    __syncthreads();
    if (ty == 0 && colact) {
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float t = 0.f;
#pragma unroll
            for (int l = 0; l < 8; ++l) t += sm[l][tx][e];
            dw_part[(int64_t)blockIdx.y * C + v * V + e] = t;
        }
    }
}

inline int row_threads(int64_t nvec) {
    int t = (int)((nvec + 31) / 32 * 32);
    return t > 256 ? 256 : (t < 32 ? 32 : t);
}

}  // namespace

cudaError_t launch_rmsnorm_fwd(bf16* out, float* rms, const bf16* inp, const bf16* w, int64_t B,
                               int64_t C, float eps, cudaStream_t s) {
    if (B == 0) return cudaSuccess;
    if (C % 8 == 0)
        rmsnorm_fwd_kernel<8><<<(unsigned)B, row_threads(C / 8), 0, s>>>(out, rms, inp, w, C, eps);
    else
        rmsnorm_fwd_kernel<1><<<(unsigned)B, row_threads(C), 0, s>>>(out, rms, inp, w, C, eps);
    return launched();
}

int rmsnorm_bwd_blocks(int64_t B) { return (int)((B + kRmsRowsPerBlock - 1) / kRmsRowsPerBlock); }

cudaError_t launch_rmsnorm_bwd(bf16* d_inp, float* d_w, float* dw_part, const bf16* grad,
                               const bf16* inp, const bf16* w, const float* rms, int64_t B,
                               int64_t C, cudaStream_t s) {
    const int nparts = rmsnorm_bwd_blocks(B);
    if (B > 0) {
        const dim3 block(32, 8);
        if (C % 8 == 0) {
            rmsnorm_bwd_dx_kernel<8><<<(unsigned)B, row_threads(C / 8), 0, s>>>(d_inp, grad, inp, w,
                                                                                rms, C);
            const dim3 grid((unsigned)((C / 8 + 31) / 32), (unsigned)nparts);
            rmsnorm_bwd_dw_kernel<8><<<grid, block, 0, s>>>(dw_part, grad, inp, rms, B, C);
        } else {
            rmsnorm_bwd_dx_kernel<1><<<(unsigned)B, row_threads(C), 0, s>>>(d_inp, grad, inp, w,
                                                                            rms, C);
            const dim3 grid((unsigned)((C + 31) / 32), (unsigned)nparts);
            rmsnorm_bwd_dw_kernel<1><<<grid, block, 0, s>>>(dw_part, grad, inp, rms, B, C);
        }
        cudaError_t e = launched(2);
        if (e != cudaSuccess) return e;
    }
    return launch_finalize(d_w, dw_part, nparts, C, nullptr, nullptr, nullptr, 0, 1, s);
}

}  // namespace mhc
