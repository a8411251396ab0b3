// Backward, pass A on the tensor cores (bf16 streams, n = 4): all per-token inner products of the
// backward from three small Gram matrices per token,
//     G [i][j] = <g_i, x_j>,   Gw[i][j] = <w * g_i, x_j>,   X2[i][j] = <x_i, x_j>
// (g = dy, w = RMSNorm weight), because every product pass A needs is a combination of them:
//     dM[i][j] = G[i][j]
//     P[i]  = <g_i, a w>  = sum_j H_pre[j]  Gw[i][j]        a = sum_j H_pre[j] x_j
//     ux[k] = <u, x_k>    = sum_i H_post[i] Gw[i][k]        u = w sum_i H_post[i] g_i
//     ax[k] = <a, x_k>    = sum_j H_pre[j]  X2[j][k]
//     s     = <u, a>      = sum_ij H_post[i] H_pre[j] Gw[i][j]
// Output, as from the scalar pass: dH[b][K] = (dH_pre, dH_post, dM), c2[b] = s / (C rho^3).
//
// One block = two tokens = the eight rows (token, stream) of x and of dy, its four warps splitting
// the columns.  Per 64 columns a thread loads 32 contiguous bytes of "its" row of dy, of x and of
// w (the four lanes of a row cover a whole 128-byte line: with 16 bytes per lane the same kernel ran
// a third slower) and issues, per 16 bytes, four m16n8k16 MMAs:
//     A rows 0-7 = dy rows, rows 8-15 = (w * dy) rows (one packed bf16 multiply per two elements),
//     B columns  = x rows                                   ->  G on top of Gw
//     A rows 0-7 = x rows (rows 8-15 zero), B = x rows      ->  X2
// Operands go from global memory straight into fragments: the reduction index of an MMA may be
// permuted freely as long as A and B agree, so the four 32-bit words of a 16-byte load feed two
// MMAs.  The scalar version of this pass spent ~430 instructions per thread and 8 columns and was
// bound by instruction issue; this one needs two dozen per 64 columns and streams at memory speed.
// Only the 4x4 blocks of the 8x8 products that pair a token with itself are used.
//
// Takes over stream_distribute_mix_backward_partials / reduce_partials and the dH part of
// rmsnorm_backward / stream_aggregate_backward of the reference
// (src/csrc/kernels/stream_ops.cuh:704-758,851-997, src/csrc/kernels/rmsnorm.cuh:233-306), with
// per-token coefficients.
#include <cuda_bf16.h>

#include "cache_hint.cuh"
#include "launch.cuh"
#include "coeffs_lanes.cuh"
#include "kernels.h"

namespace mhc {

namespace {

constexpr int kGWarps = 4;
constexpr int kGBatch = 3;   // chunks of 64 columns whose loads are in flight together

__device__ __forceinline__ void g_mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t g_mul_bf16x2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&a),
                                     *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}

// FUSE: the block also runs the backward of its two tokens' coefficients (coeffs_lanes.cuh) on
// warp 0 once the inner products are known, instead of leaving dH to a second kernel.
template <bool FUSE>
__global__ void __launch_bounds__(kGWarps * 32, 6)
bwd_gram_kernel(float* __restrict__ dH, float* __restrict__ c2out, const bf16* __restrict__ x,
                const bf16* __restrict__ g, const bf16* __restrict__ w,
                const float* __restrict__ H_pre, const float* __restrict__ H_post,
                const float* __restrict__ rms, int64_t B, int64_t C, int coef_stride,
                const GramFuse f) {
    __shared__ float part[kGWarps][2][3][16];   // [warp][token][G, Gw, X2][i*4+j]
    __shared__ float tot[2][3][16];
    __shared__ float coef[2][12];               // hp[4] hq[4] 1/rho
    __shared__ float dHs[2][24];                // FUSE: the tokens' dH and c2 stay in the block
    __shared__ float c2s[2];
    __shared__ float pts[2][28];                // FUSE: the tokens' terms of d_bias and d_alpha
    extern __shared__ __align__(16) float den[];   // FUSE: [2 tokens][2*iters][4] saved denominators
    pdl_trigger();   // the dx pass that follows may fetch its phi fragments while this kernel drains
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int gq = lane >> 2, q = lane & 3;     // fragment row / column group
    const int64_t pair = blockIdx.x;
    const int64_t row = pair * 8 + gq;          // row (token, stream) of the [B*4, C] views
    const bool valid = row < B * 4;             // an odd B leaves the last block one token short
    const bf16* xr = x + (valid ? row : 0) * C;
    const bf16* gr = g + (valid ? row : 0) * C;

    // the coefficients go first: small loads issued behind the row traffic wait for it
    if (tid < 18) {
        const int t = tid / 9, k = tid % 9;
        const int64_t b = pair * 2 + t;
        float v = 0.f;
        if (b < B) {
            const int64_t cb = b * coef_stride;
            v = k < 4 ? H_pre[cb * 4 + k] : k < 8 ? H_post[cb * 4 + (k - 4)] : 1.f / rms[b];
        }
        coef[t][k] = v;
    }

    // FUSE: what the coefficient backward needs besides dH is fetched now as well
    const int tl = lane >> 4, e = lane & 15;    // warp 0: token slot and matrix element of a lane
    const int64_t tokf = pair * 2 + tl;
    LaneIn lin{0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    float rh = 1.f, al0 = 0.f, al1 = 0.f, al2 = 0.f;
    if constexpr (FUSE) {
        const int dpt = 2 * f.iters * 4;
        const int64_t base = pair * 2 * dpt, lim = B * dpt;
        for (int k = tid; k < 2 * dpt; k += kGWarps * 32)
            den[k] = (base + k < lim) ? f.sk_den[base + k] : 1.f;
        if (tid < 56) (&pts[0][0])[tid] = 0.f;
        if (warp == 0 && tokf < B) {
            lin.m = f.M[tokf * 16 + e];
            lin.p_res = f.proj[tokf * 24 + 8 + e];
            if (e < 8) {
                lin.h = e < 4 ? H_pre[tokf * 4 + e] : H_post[tokf * 4 + (e - 4)];
                lin.p_e = f.proj[tokf * 24 + e];
            }
            rh = f.rms_h[tokf];
            al0 = f.alpha[0];
            al1 = f.alpha[1];
            al2 = f.alpha[2];
        }
    }

    float acc1[4] = {0.f, 0.f, 0.f, 0.f}, acc2[4] = {0.f, 0.f, 0.f, 0.f};
    // 64 columns at a time: the four lanes of a row take 32 contiguous bytes each, so a warp's pair
    // of loads covers whole 128-byte lines of its eight rows
    const int nchunk = (int)(C / 64);
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const uint64_t keep = l2_evict_last();   // x and dy are read once more, by the dx pass
    for (int c0 = warp; c0 < nchunk; c0 += kGWarps * kGBatch) {
        uint4 gv[kGBatch][2], xv[kGBatch][2];
#pragma unroll
        for (int u = 0; u < kGBatch; ++u) {
            const int c = c0 + u * kGWarps;
            const bool in = c < nchunk && valid;
            const int64_t off = (int64_t)c * 64 + 16 * q;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                gv[u][e] = in ? ldg_stream_hint(gr + off + 8 * e, keep) : zero;
                xv[u][e] = in ? ldg_stream_hint(xr + off + 8 * e, keep) : zero;
            }
        }
#pragma unroll
        for (int u = 0; u < kGBatch; ++u) {
            const int c = c0 + u * kGWarps;
            if (c >= nchunk) break;
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint4 wv = *reinterpret_cast<const uint4*>(w + (int64_t)c * 64 + 16 * q + 8 * e);
                const uint4 gg = gv[u][e], xx = xv[u][e];
                const uint32_t gw0 = g_mul_bf16x2(gg.x, wv.x), gw1 = g_mul_bf16x2(gg.y, wv.y);
                const uint32_t gw2 = g_mul_bf16x2(gg.z, wv.z), gw3 = g_mul_bf16x2(gg.w, wv.w);
                g_mma_16816(acc1, gg.x, gw0, gg.y, gw1, xx.x, xx.y);
                g_mma_16816(acc1, gg.z, gw2, gg.w, gw3, xx.z, xx.w);
                g_mma_16816(acc2, xx.x, 0u, xx.y, 0u, xx.x, xx.y);
                g_mma_16816(acc2, xx.z, 0u, xx.w, 0u, xx.z, xx.w);
            }
        }
    }
    // accumulator element (row gq, columns 2q, 2q+1): row = (token gq/4, stream gq%4), column =
    // (token q/2, stream 2(q%2) [+1]); kept where the two tokens agree
    if ((gq >> 2) == (q >> 1)) {
        const int t = gq >> 2, i = gq & 3, j = 2 * (q & 1);
        part[warp][t][0][i * 4 + j] = acc1[0];
        part[warp][t][0][i * 4 + j + 1] = acc1[1];
        part[warp][t][1][i * 4 + j] = acc1[2];
        part[warp][t][1][i * 4 + j + 1] = acc1[3];
        part[warp][t][2][i * 4 + j] = acc2[0];
        part[warp][t][2][i * 4 + j + 1] = acc2[1];
    }
    __syncthreads();
    if (tid < 96) {
        float v = 0.f;
#pragma unroll
        for (int wi = 0; wi < kGWarps; ++wi) v += (&part[wi][0][0][0])[tid];
        (&tot[0][0][0])[tid] = v;
    }
    __syncthreads();
    if (tid < 48) {
        const int t = tid / 24, k = tid % 24;
        const int64_t b = pair * 2 + t;
        if (b < B) {
            const float* G = tot[t][0];
            const float* Gw = tot[t][1];
            const float* X2 = tot[t][2];
            const float* hp = coef[t];
            const float* hq = coef[t] + 4;
            const float ri = coef[t][8];
            float s = 0.f;
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) s = fmaf(hq[i] * hp[j], Gw[i * 4 + j], s);
            const float c2 = s * ri * ri * ri / (float)C;
            if (k == 0) c2out[b] = c2;
            float o;
            if (k < 4) {
                float ux = 0.f, ax = 0.f;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    ux = fmaf(hq[i], Gw[i * 4 + k], ux);
                    ax = fmaf(hp[i], X2[i * 4 + k], ax);
                }
                o = ri * ux - c2 * ax;
            } else if (k < 8) {
                float P = 0.f;
#pragma unroll
                for (int j = 0; j < 4; ++j) P = fmaf(hp[j], Gw[(k - 4) * 4 + j], P);
                o = P * ri;
            } else {
                o = G[k - 8];
            }
            if constexpr (FUSE) {
                dHs[t][k] = o;
                if (k == 0) c2s[t] = c2;
            } else {
                dH[b * 24 + k] = o;
            }
        }
    }
    if constexpr (FUSE) {
        __syncthreads();
        if (warp == 0) {
            const bool act = tokf < B;
            if (act) {
                lin.dres = dHs[tl][8 + e];
                if (e < 8) lin.dh = dHs[tl][e];
            }
            coeffs_lanes_token(tokf, act, e, 4, 4 * C, f.iters, B, lin, rh, al0, al1, al2,
                               coef[tl][8], act ? c2s[tl] : 0.f, den + tl * 2 * f.iters * 4, pts[tl],
                               f.dpr, f.qq, f.mo);
            __syncwarp();
            if (lane < 27) f.partials[(int64_t)pair * 27 + lane] = pts[0][lane] + pts[1][lane];
        }
    }
}

}  // namespace

bool bwd_gram_supported(Dims d) { return d.n == 4 && d.C % 64 == 0; }

// two tokens per block, up to the batch rounded to 16 tokens: the fused variant also zeroes the
// padding columns of the transposed bf16 copy of dpr that the next pass reads
int bwd_gram_blocks(Dims d) { return (int)((d.B + 15) / 16 * 8); }

cudaError_t launch_bwd_gram(float* dH, float* c2, const bf16* x, const bf16* g, const bf16* w,
                            const float* H_pre, const float* H_post, int coef_stride,
                            const float* rms, Dims d, cudaStream_t s, const GramFuse* fuse) {
    if (d.B == 0) return cudaSuccess;
    if (!bwd_gram_supported(d)) return cudaErrorNotSupported;
    const unsigned grid = (unsigned)bwd_gram_blocks(d);
    if (fuse != nullptr) {
        const size_t smem = (size_t)2 * 2 * fuse->iters * 4 * sizeof(float);
        if (smem > 40 * 1024) return cudaErrorNotSupported;
        bwd_gram_kernel<true><<<grid, kGWarps * 32, smem, s>>>(dH, c2, x, g, w, H_pre, H_post, rms,
                                                               d.B, d.C, coef_stride, *fuse);
    } else {
        bwd_gram_kernel<false><<<grid, kGWarps * 32, 0, s>>>(dH, c2, x, g, w, H_pre, H_post, rms, d.B,
                                                             d.C, coef_stride, GramFuse());
    }
    return launched();
}

}  // namespace mhc
