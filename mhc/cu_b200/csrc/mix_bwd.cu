// Backward, pass A: all per-token inner products the backward needs, one block per token.
//
// Thread 0 starts two bulk async copies (TMA, cp.async.bulk) — the token's [n, C] blocks of x and
// of dy — into shared memory; the block then makes ONE sweep over them accumulating
//     s = <u, a>,  dM[i,j] = <g_i, x_j>,  P[i] = <g_i, a*w>,  ux[i] = <u, x_i>,  ax[i] = <a, x_i>
// (u = w * sum_i H_post[i] g_i,  a = sum_i H_pre[i] x_i) and reduces them over the block.  The
// warp-level reduction is a reduce-scatter (31 shuffles for 32 values instead of 5 per value).
// Output, as before: dH[b][K] = (dH_pre, dH_post, dM) and c2[b] = s / (C rho^3).
//
// Takes over stream_distribute_mix_backward_partials / reduce_partials and the dH part of
// rmsnorm_backward / stream_aggregate_backward of the reference
// (src/csrc/kernels/stream_ops.cuh:704-758,851-997, src/csrc/kernels/rmsnorm.cuh:233-306), with
// per-token coefficients.
#include "async.cuh"
#include "kernels.h"

namespace mhc {

namespace {

// Sum 32 per-lane values over the warp; on return lane L holds the total of r[L] (in r[0]).
__device__ __forceinline__ float warp_reduce_scatter32(float (&r)[32]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < off; ++i) {
            const float send = upper ? r[i] : r[i + off];
            const float keep = upper ? r[i + off] : r[i];
            r[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
        }
    }
    return r[0];
}

template <typename T>
struct RedParams {
    float* dH;
    float* c2;
    const T* x;
    const T* g;
    const bf16* w;
    const float* H_pre;
    const float* H_post;
    const float* rms;
    int* status;
    int64_t C;
    int n;
    int coef_stride;
};

template <typename T, int V, int MAXN>
__global__ void __launch_bounds__(256)
bwd_reduce_staged_kernel(const RedParams<T> p) {
    constexpr int NR = 1 + MAXN * MAXN + 3 * MAXN;
    constexpr int NCH = (NR + 31) / 32;       // chunks of 32 values for the reduce-scatter
    constexpr int OM = 1, OP = 1 + MAXN * MAXN, OU = OP + MAXN, OA = OU + MAXN;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    const int n = p.n;
    const int64_t C = p.C;
    const int64_t b = blockIdx.x;
    const uint32_t row_bytes = (uint32_t)(n * C * sizeof(T));
    const uint32_t row_pad = (row_bytes + 127) & ~127u;
    T* xs = reinterpret_cast<T*>(smem_raw);
    T* gs = reinterpret_cast<T*>(smem_raw + row_pad);
    float* red = reinterpret_cast<float*>(smem_raw + 2 * row_pad);   // [8 warps][NCH*32]
    float* tot = red + 8 * NCH * 32;                                   // [NCH*32]
    uint64_t* bar = reinterpret_cast<uint64_t*>(tot + NCH * 32);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = blockDim.x >> 5;

    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
        mbar_arrive_expect_tx(bar, 2 * row_bytes);
        bulk_copy_g2s(xs, p.x + b * n * C, row_bytes, bar);
        bulk_copy_g2s(gs, p.g + b * n * C, row_bytes, bar);
    }
    __syncthreads();   // nobody may poll the barrier before it is initialised
    const int64_t cb = b * p.coef_stride;
    float hp[MAXN], hq[MAXN];
#pragma unroll
    for (int i = 0; i < MAXN; ++i) {
        hp[i] = (i < n) ? p.H_pre[cb * n + i] : 0.f;
        hq[i] = (i < n) ? p.H_post[cb * n + i] : 0.f;
    }
    const float ri = 1.f / p.rms[b];

    const int ok = __syncthreads_and(mbar_wait_bounded(bar, 0) ? 1 : 0);
    if (!ok) {
        if (tid == 0 && p.status != nullptr) atomicOr(p.status, kDevErrBulkWait);
        return;
    }

    float acc[NCH * 32];
#pragma unroll
    for (int k = 0; k < NCH * 32; ++k) acc[k] = 0.f;

    const int64_t nvec = C / V;
    for (int64_t v = tid; v < nvec; v += blockDim.x) {
        float xv[MAXN][V], gv[MAXN][V], wv[V];
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                load_vec<V>(xs + i * C + v * V, xv[i]);
                load_vec<V>(gs + i * C + v * V, gv[i]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) { xv[i][e] = 0.f; gv[i][e] = 0.f; }
            }
        }
        load_weight<V>(p.w, v * V, wv);
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float a = 0.f, dyh = 0.f;
#pragma unroll
            for (int i = 0; i < MAXN; ++i) {
                a = fmaf(hp[i], xv[i][e], a);
                dyh = fmaf(hq[i], gv[i][e], dyh);
            }
            const float u = dyh * wv[e];
            const float aw = a * wv[e];
            acc[0] = fmaf(u, a, acc[0]);
#pragma unroll
            for (int i = 0; i < MAXN; ++i) {
                acc[OP + i] = fmaf(gv[i][e], aw, acc[OP + i]);
                acc[OU + i] = fmaf(u, xv[i][e], acc[OU + i]);
                acc[OA + i] = fmaf(a, xv[i][e], acc[OA + i]);
#pragma unroll
                for (int j = 0; j < MAXN; ++j)
                    acc[OM + i * MAXN + j] = fmaf(gv[i][e], xv[j][e], acc[OM + i * MAXN + j]);
            }
        }
    }
    // warp reduce-scatter chunk by chunk, then add the warps in order
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
        float r[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) r[k] = acc[c * 32 + k];
        red[(warp * NCH + c) * 32 + lane] = warp_reduce_scatter32(r);
    }
    __syncthreads();
    for (int k = tid; k < NCH * 32; k += blockDim.x) {
        float t = 0.f;
        for (int wi = 0; wi < nwarps; ++wi) t += red[wi * NCH * 32 + k];
        tot[k] = t;
    }
    __syncthreads();
    const float c2 = tot[0] * ri * ri * ri / (float)C;
    if (tid == 0) p.c2[b] = c2;
    const int K = 2 * n + n * n;
    for (int k = tid; k < K; k += blockDim.x) {
        float o;
        if (k < n) {
            o = ri * tot[OU + k] - c2 * tot[OA + k];
        } else if (k < 2 * n) {
            o = tot[OP + (k - n)] * ri;
        } else {
            const int e = k - 2 * n;
            o = tot[OM + (e / n) * MAXN + (e % n)];
        }
        p.dH[b * K + k] = o;
    }
}

}  // namespace

static size_t reduce_smem(Dims d, size_t elem, int maxn) {
    const size_t row = ((size_t)d.n * d.C * elem + 127) & ~size_t(127);
    const int NR = 1 + maxn * maxn + 3 * maxn;
    const int NCH = (NR + 31) / 32;
    return 2 * row + (size_t)(8 + 1) * NCH * 32 * 4 + 16;
}

bool bwd_reduce_staged_supported(Dims d, size_t elem) {
    const int V = (int)(16 / elem);
    if (d.n > 8 || d.C % V != 0) return false;
    return reduce_smem(d, elem, 8) <= 100 * 1024;
}

template <typename T>
cudaError_t launch_bwd_reduce_staged(float* dH, float* c2, const T* x, const T* g, const bf16* w,
                                     const float* H_pre, const float* H_post, int coef_stride,
                                     const float* rms, int* status, Dims d, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!bwd_reduce_staged_supported(d, sizeof(T))) return cudaErrorNotSupported;
    constexpr int V = VecWidth<T>::value;
    RedParams<T> p{dH, c2, x, g, w, H_pre, H_post, rms, status, d.C, d.n, coef_stride};
    const int64_t nvec = d.C / V;
    // two vectors per thread where the row is long enough, at most 8 warps
    int threads = (int)(((nvec + 1) / 2 + 31) / 32 * 32);
    if (threads < 32) threads = 32;
    if (threads > 256) threads = 256;
    const unsigned grid = (unsigned)d.B;
    cudaError_t e;
    if (d.n <= 4) {
        auto k = bwd_reduce_staged_kernel<T, V, 4>;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        if (e != cudaSuccess) return e;
        k<<<grid, threads, reduce_smem(d, sizeof(T), 4), s>>>(p);
    } else {
        auto k = bwd_reduce_staged_kernel<T, V, 8>;
        e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 110 * 1024);
        if (e != cudaSuccess) return e;
        k<<<grid, threads, reduce_smem(d, sizeof(T), 8), s>>>(p);
    }
    return launched();
}

template cudaError_t launch_bwd_reduce_staged<float>(float*, float*, const float*, const float*,
                                                     const bf16*, const float*, const float*, int,
                                                     const float*, int*, Dims, cudaStream_t);
template cudaError_t launch_bwd_reduce_staged<bf16>(float*, float*, const bf16*, const bf16*,
                                                    const bf16*, const float*, const float*, int,
                                                    const float*, int*, Dims, cudaStream_t);

}  // namespace mhc
