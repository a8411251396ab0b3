// The dynamic-H layer in two halves, for callers that run their own sub-layer F between them
// (a transformer block: y_hat -> attention / MLP -> f):
//
//   pre :  coefficients, then  y_hat[b,:] = (sum_i H_pre[i] x[i,:]) / rho * w            [B, C]
//   post:  y[i,:] = sum_j M[i,j] x[j,:] + H_post[i] f[b,:]                               [B, n, C]
//
// and their backward passes (post: d_f, dH_post, dM and the M^T dy part of dx; pre: from d_y_hat and
// the coefficient gradients dH_post / dM coming back from post, the rest of dx and all parameter
// gradients).  The reference layer is monolithic (src/python/mhc/layer.py:61-101,
// src/python/bindings.cu:403-481) and has no hook between aggregate+norm and distribute+mix; these
// kernels split its stream_aggregate / rmsnorm / stream_distribute_mix steps
// (src/csrc/kernels/stream_ops.cuh:44-330, src/csrc/kernels/rmsnorm.cuh) at that point.  n <= 8,
// fp32 or bf16 streams, C a multiple of the 16-byte vector.  One block per token; plain vector
// loads (these are first, correct versions: they are not on the benchmarked path).
#include "kernels.h"

namespace mhc {

namespace {

constexpr int kSplitThreads = 128;

template <int NV>
__device__ __forceinline__ void block_sum(float (&v)[NV], float* red /* [warps][NV] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        float t = v[k];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) red[warp * NV + k] = t;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        float t = 0.f;
        for (int w = 0; w < nw; ++w) t += red[w * NV + k];
        v[k] = t;
    }
    __syncthreads();
}

// ---- pre forward: y_hat and rho from x and H_pre --------------------------------------------------
template <typename T, int V, int MAXN>
__global__ void __launch_bounds__(kSplitThreads)
pre_apply_kernel(T* __restrict__ yhat, float* __restrict__ rho, const T* __restrict__ x,
                 const bf16* __restrict__ w, const float* __restrict__ H_pre, int n, int64_t C,
                 float eps) {
    __shared__ float red[kSplitThreads / 32];
    const int64_t b = blockIdx.x;
    float hp[MAXN];
#pragma unroll
    for (int i = 0; i < MAXN; ++i) hp[i] = (i < n) ? H_pre[b * n + i] : 0.f;
    const T* xb = x + b * n * C;
    const int64_t nvec = C / V;
    float ss[1] = {0.f};
    for (int64_t v = threadIdx.x; v < nvec; v += kSplitThreads) {
        float a[V];
#pragma unroll
        for (int e = 0; e < V; ++e) a[e] = 0.f;
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                float xv[V];
                load_vec<V>(xb + i * C + v * V, xv);
#pragma unroll
                for (int e = 0; e < V; ++e) a[e] = fmaf(hp[i], xv[e], a[e]);
            }
        }
#pragma unroll
        for (int e = 0; e < V; ++e) ss[0] = fmaf(a[e], a[e], ss[0]);
    }
    block_sum<1>(ss, red);
    const float r = sqrtf(ss[0] / (float)C + eps);
    const float ri = 1.f / r;
    if (threadIdx.x == 0) rho[b] = r;
    for (int64_t v = threadIdx.x; v < nvec; v += kSplitThreads) {
        float a[V], wv[V];
#pragma unroll
        for (int e = 0; e < V; ++e) a[e] = 0.f;
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                float xv[V];
                load_vec<V>(xb + i * C + v * V, xv);
#pragma unroll
                for (int e = 0; e < V; ++e) a[e] = fmaf(hp[i], xv[e], a[e]);
            }
        }
        load_weight<V>(w, v * V, wv);
#pragma unroll
        for (int e = 0; e < V; ++e) a[e] = a[e] * ri * wv[e];
        store_vec<V>(yhat + b * C + v * V, a);
    }
}

// ---- post forward -----------------------------------------------------------------------------------
template <typename T, int V, int MAXN>
__global__ void __launch_bounds__(kSplitThreads)
post_fwd_kernel(T* __restrict__ y, const T* __restrict__ x, const T* __restrict__ f,
                const float* __restrict__ H_post, const float* __restrict__ M, int n, int64_t C) {
    const int64_t b = blockIdx.x;
    float hq[MAXN], m[MAXN][MAXN];
#pragma unroll
    for (int i = 0; i < MAXN; ++i) {
        hq[i] = (i < n) ? H_post[b * n + i] : 0.f;
#pragma unroll
        for (int j = 0; j < MAXN; ++j) m[i][j] = (i < n && j < n) ? M[b * n * n + i * n + j] : 0.f;
    }
    const T* xb = x + b * n * C;
    T* yb = y + b * n * C;
    const int64_t nvec = C / V;
    for (int64_t v = threadIdx.x; v < nvec; v += kSplitThreads) {
        float xv[MAXN][V], fv[V];
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                load_vec<V>(xb + i * C + v * V, xv[i]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) xv[i][e] = 0.f;
            }
        }
        load_vec<V>(f + b * C + v * V, fv);
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                float o[V];
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float t = hq[i] * fv[e];
#pragma unroll
                    for (int j = 0; j < MAXN; ++j) t = fmaf(m[i][j], xv[j][e], t);
                    o[e] = t;
                }
                store_vec<V>(yb + i * C + v * V, o);
            }
        }
    }
}

// ---- post backward: d_f, dx_part = M^T dy, dH_post[i] = <dy_i, f>, dM[i,j] = <dy_i, x_j> -------------
template <typename T, int V, int MAXN>
__global__ void __launch_bounds__(kSplitThreads)
post_bwd_kernel(T* __restrict__ dx_part, T* __restrict__ d_f, float* __restrict__ dH_post,
                float* __restrict__ dM, const T* __restrict__ g, const T* __restrict__ x,
                const T* __restrict__ f, const float* __restrict__ H_post,
                const float* __restrict__ M, int n, int64_t C) {
    constexpr int NV = MAXN + MAXN * MAXN;
    __shared__ float red[(kSplitThreads / 32) * NV];
    const int64_t b = blockIdx.x;
    float hq[MAXN], m[MAXN][MAXN], acc[NV];
#pragma unroll
    for (int i = 0; i < MAXN; ++i) {
        hq[i] = (i < n) ? H_post[b * n + i] : 0.f;
#pragma unroll
        for (int j = 0; j < MAXN; ++j) m[i][j] = (i < n && j < n) ? M[b * n * n + i * n + j] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) acc[k] = 0.f;
    const T* xb = x + b * n * C;
    const T* gb = g + b * n * C;
    const int64_t nvec = C / V;
    for (int64_t v = threadIdx.x; v < nvec; v += kSplitThreads) {
        float xv[MAXN][V], gv[MAXN][V], fv[V];
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                load_vec<V>(xb + i * C + v * V, xv[i]);
                load_vec<V>(gb + i * C + v * V, gv[i]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) { xv[i][e] = 0.f; gv[i][e] = 0.f; }
            }
        }
        load_vec<V>(f + b * C + v * V, fv);
        float df[V];
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float t = 0.f;
#pragma unroll
            for (int i = 0; i < MAXN; ++i) {
                t = fmaf(hq[i], gv[i][e], t);
                acc[i] = fmaf(gv[i][e], fv[e], acc[i]);
#pragma unroll
                for (int j = 0; j < MAXN; ++j)
                    acc[MAXN + i * MAXN + j] = fmaf(gv[i][e], xv[j][e], acc[MAXN + i * MAXN + j]);
            }
            df[e] = t;
        }
        store_vec<V>(d_f + b * C + v * V, df);
#pragma unroll
        for (int j = 0; j < MAXN; ++j) {
            if (j < n) {
                float o[V];
#pragma unroll
                for (int e = 0; e < V; ++e) {
                    float t = 0.f;
#pragma unroll
                    for (int i = 0; i < MAXN; ++i) t = fmaf(m[i][j], gv[i][e], t);
                    o[e] = t;
                }
                store_vec<V>(dx_part + b * n * C + j * C + v * V, o);
            }
        }
    }
    block_sum<NV>(acc, red);
    if (threadIdx.x < n) dH_post[b * n + threadIdx.x] = acc[threadIdx.x];
    if (threadIdx.x < n * n) {
        const int i = threadIdx.x / n, j = threadIdx.x % n;
        dM[b * n * n + threadIdx.x] = acc[MAXN + i * MAXN + j];
    }
}

// ---- pre backward, pass A: c2 and dH_pre from d_y_hat; assembles the dH row the coefficient
//      backward consumes: (dH_pre | dH_post | dM) -----------------------------------------------------------
template <typename T, int V, int MAXN>
__global__ void __launch_bounds__(kSplitThreads)
pre_bwd_reduce_kernel(float* __restrict__ dH, float* __restrict__ c2, const T* __restrict__ dyh,
                      const T* __restrict__ x, const bf16* __restrict__ w,
                      const float* __restrict__ H_pre, const float* __restrict__ rho,
                      const float* __restrict__ dH_post, const float* __restrict__ dM, int n,
                      int64_t C) {
    constexpr int NV = 1 + 2 * MAXN;   // s = <u, a>, ux[j] = <u, x_j>, ax[j] = <a, x_j>
    __shared__ float red[(kSplitThreads / 32) * NV];
    const int64_t b = blockIdx.x;
    float hp[MAXN], acc[NV];
#pragma unroll
    for (int i = 0; i < MAXN; ++i) hp[i] = (i < n) ? H_pre[b * n + i] : 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) acc[k] = 0.f;
    const T* xb = x + b * n * C;
    const int64_t nvec = C / V;
    for (int64_t v = threadIdx.x; v < nvec; v += kSplitThreads) {
        float xv[MAXN][V], dv[V], wv[V];
#pragma unroll
        for (int i = 0; i < MAXN; ++i) {
            if (i < n) {
                load_vec<V>(xb + i * C + v * V, xv[i]);
            } else {
#pragma unroll
                for (int e = 0; e < V; ++e) xv[i][e] = 0.f;
            }
        }
        load_vec<V>(dyh + b * C + v * V, dv);
        load_weight<V>(w, v * V, wv);
#pragma unroll
        for (int e = 0; e < V; ++e) {
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < MAXN; ++i) a = fmaf(hp[i], xv[i][e], a);
            const float u = dv[e] * wv[e];
            acc[0] = fmaf(u, a, acc[0]);
#pragma unroll
            for (int j = 0; j < MAXN; ++j) {
                acc[1 + j] = fmaf(u, xv[j][e], acc[1 + j]);
                acc[1 + MAXN + j] = fmaf(a, xv[j][e], acc[1 + MAXN + j]);
            }
        }
    }
    block_sum<NV>(acc, red);
    const float ri = 1.f / rho[b];
    const float c2b = acc[0] * ri * ri * ri / (float)C;
    const int K = 2 * n + n * n;
    if (threadIdx.x == 0) c2[b] = c2b;
    if (threadIdx.x < n) {
        const int j = threadIdx.x;
        dH[b * K + j] = ri * acc[1 + j] - c2b * acc[1 + MAXN + j];
        dH[b * K + n + j] = dH_post[b * n + j];
    }
    if (threadIdx.x < n * n) dH[b * K + 2 * n + threadIdx.x] = dM[b * n * n + threadIdx.x];
}

template <typename T>
struct SplitVec { static constexpr int value = 16 / sizeof(T); };

}  // namespace

bool split_ops_supported(Dims d, size_t elem) { return d.n <= 8 && d.C % (int64_t)(16 / elem) == 0; }

#define MHC_SPLIT_DISPATCH(KERNEL, ...)                                                        \
    do {                                                                                       \
        constexpr int V = SplitVec<T>::value;                                                  \
        if (d.n <= 4) KERNEL<T, V, 4><<<(unsigned)d.B, kSplitThreads, 0, s>>>(__VA_ARGS__);     \
        else KERNEL<T, V, 8><<<(unsigned)d.B, kSplitThreads, 0, s>>>(__VA_ARGS__);              \
    } while (0)

template <typename T>
cudaError_t launch_pre_apply(T* yhat, float* rho, const T* x, const bf16* w, const float* H_pre,
                             Dims d, float eps, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!split_ops_supported(d, sizeof(T))) return cudaErrorNotSupported;
    MHC_SPLIT_DISPATCH(pre_apply_kernel, yhat, rho, x, w, H_pre, d.n, d.C, eps);
    return launched();
}

template <typename T>
cudaError_t launch_post_fwd(T* y, const T* x, const T* f, const float* H_post, const float* M,
                            Dims d, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!split_ops_supported(d, sizeof(T))) return cudaErrorNotSupported;
    MHC_SPLIT_DISPATCH(post_fwd_kernel, y, x, f, H_post, M, d.n, d.C);
    return launched();
}

template <typename T>
cudaError_t launch_post_bwd(T* dx_part, T* d_f, float* dH_post, float* dM, const T* g, const T* x,
                            const T* f, const float* H_post, const float* M, Dims d,
                            cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!split_ops_supported(d, sizeof(T))) return cudaErrorNotSupported;
    MHC_SPLIT_DISPATCH(post_bwd_kernel, dx_part, d_f, dH_post, dM, g, x, f, H_post, M, d.n, d.C);
    return launched();
}

template <typename T>
cudaError_t launch_pre_bwd_reduce(float* dH, float* c2, const T* dyh, const T* x, const bf16* w,
                                  const float* H_pre, const float* rho, const float* dH_post,
                                  const float* dM, Dims d, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!split_ops_supported(d, sizeof(T))) return cudaErrorNotSupported;
    MHC_SPLIT_DISPATCH(pre_bwd_reduce_kernel, dH, c2, dyh, x, w, H_pre, rho, dH_post, dM, d.n, d.C);
    return launched();
}

#define MHC_SPLIT_INST(T)                                                                          \
    template cudaError_t launch_pre_apply<T>(T*, float*, const T*, const bf16*, const float*, Dims, \
                                             float, cudaStream_t);                                 \
    template cudaError_t launch_post_fwd<T>(T*, const T*, const T*, const float*, const float*,    \
                                            Dims, cudaStream_t);                                   \
    template cudaError_t launch_post_bwd<T>(T*, T*, float*, float*, const T*, const T*, const T*,  \
                                            const float*, const float*, Dims, cudaStream_t);       \
    template cudaError_t launch_pre_bwd_reduce<T>(float*, float*, const T*, const T*, const bf16*, \
                                                  const float*, const float*, const float*,        \
                                                  const float*, Dims, cudaStream_t);
MHC_SPLIT_INST(float)
MHC_SPLIT_INST(bf16)

}  // namespace mhc
