// d_phi of the bf16 backward on mma.sync tensor-core tiles, as a pass of its own:
//
//   dphi_mma  dphi[k,m] = sum_b dpr[b,k] x[b,m]: A = dpr^T, B = x with token pairs interleaved in
//             registers (PRMT), one block owns 64 columns for all tokens, so dphi is written once,
//             in a fixed summation order.
//
// It reads a small bf16 copy of dpr, dprT[KP][Bp] (k major), KP = K rounded up to 8, Bp = B rounded
// up to 16.  The monolithic layer gets d_phi from the fused dx / d_phi sweep (bwd_fused.cu); this
// kernel serves the first half of the split layer, whose dx pass has no tensor-core part.
//
// Takes over the eager GEMM d_phi = d_p^T @ x_flat of the reference's dynamic backward
// (src/python/mhc/ops.py:330-349).
#include "kernels.h"

namespace mhc {

namespace {

__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t ldg_u32(const bf16* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}

// ------------------------------------------------------------------------------------------------
// dphi.  Block = 8 warps x 64 flat columns; MT16 = m16 row tiles of dphi handled (blockIdx.y picks
// the group).  Warps take token groups round-robin and are summed through shared memory in warp
// order.
constexpr int kDphiWarps = 8;
constexpr int kDphiCols = 64;

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

template <int MT16>
__global__ void __launch_bounds__(kDphiWarps * 32)
dphi_mma_kernel(float* __restrict__ dphi, const bf16* __restrict__ x,
                const bf16* __restrict__ dprT, int64_t B, int64_t Bp, int K, int KP, int64_t nC) {
    __shared__ float sred[kDphiWarps][16][kDphiCols];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int64_t col0 = (int64_t)blockIdx.x * kDphiCols;
    const int row0 = blockIdx.y * MT16 * 16;
    const bool colin = (col0 + 8 * g) < nC;

    float acc[MT16][8][4];
#pragma unroll
    for (int m = 0; m < MT16; ++m)
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][u][e] = 0.f;

    const int64_t ngroups = (B + 15) / 16;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const bf16* xcol = x + col0 + 8 * g;
    // operands of one token group: four x vectors (tokens ta, ta+1, ta+8, ta+9) and the A fragments
    struct Operands {
        uint4 xa, xb, xc, xd;
        uint32_t afr[MT16][4];
    };
    auto fetch = [&](int64_t grp, Operands& o) {
        const int64_t ta = grp * 16 + 2 * q;
        o.xa = zero; o.xb = zero; o.xc = zero; o.xd = zero;
        if (colin) {
            if (ta < B) o.xa = *reinterpret_cast<const uint4*>(xcol + ta * nC);
            if (ta + 1 < B) o.xb = *reinterpret_cast<const uint4*>(xcol + (ta + 1) * nC);
            if (ta + 8 < B) o.xc = *reinterpret_cast<const uint4*>(xcol + (ta + 8) * nC);
            if (ta + 9 < B) o.xd = *reinterpret_cast<const uint4*>(xcol + (ta + 9) * nC);
        }
#pragma unroll
        for (int m = 0; m < MT16; ++m) {
            const int r0 = row0 + 16 * m + g, r1 = r0 + 8;
            o.afr[m][0] = (r0 < KP) ? ldg_u32(dprT + (int64_t)r0 * Bp + ta) : 0u;
            o.afr[m][1] = (r1 < KP) ? ldg_u32(dprT + (int64_t)r1 * Bp + ta) : 0u;
            o.afr[m][2] = (r0 < KP) ? ldg_u32(dprT + (int64_t)r0 * Bp + ta + 8) : 0u;
            o.afr[m][3] = (r1 < KP) ? ldg_u32(dprT + (int64_t)r1 * Bp + ta + 8) : 0u;
        }
    };
    Operands cur, nxt;
    if (warp < ngroups) fetch(warp, cur);
    for (int64_t grp = warp; grp < ngroups; grp += kDphiWarps) {
        // the next group's loads are in flight while this group's MMAs run
        const bool more = grp + kDphiWarps < ngroups;
        if (more) fetch(grp + kDphiWarps, nxt);
        const uint32_t wa[4] = {cur.xa.x, cur.xa.y, cur.xa.z, cur.xa.w};
        const uint32_t wb[4] = {cur.xb.x, cur.xb.y, cur.xb.z, cur.xb.w};
        const uint32_t wc[4] = {cur.xc.x, cur.xc.y, cur.xc.z, cur.xc.w};
        const uint32_t wd[4] = {cur.xd.x, cur.xd.y, cur.xd.z, cur.xd.w};
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            // columns 2p and 2p+1 of this thread's 8: (token ta, ta+1) and (ta+8, ta+9) pairs
            const uint32_t b0e = prmt(wa[p], wb[p], 0x5410), b0o = prmt(wa[p], wb[p], 0x7632);
            const uint32_t b1e = prmt(wc[p], wd[p], 0x5410), b1o = prmt(wc[p], wd[p], 0x7632);
#pragma unroll
            for (int m = 0; m < MT16; ++m) {
                mma_16816(acc[m][2 * p], cur.afr[m][0], cur.afr[m][1], cur.afr[m][2],
                          cur.afr[m][3], b0e, b1e);
                mma_16816(acc[m][2 * p + 1], cur.afr[m][0], cur.afr[m][1], cur.afr[m][2],
                          cur.afr[m][3], b0o, b1o);
            }
        }
        if (more) cur = nxt;
    }
    // acc[m][u][0..1] -> row 16m+g, columns 16q+u and 16q+8+u; acc[m][u][2..3] -> row 16m+g+8.
    // One m16 tile at a time goes through shared memory and is summed over the warps in order.
#pragma unroll
    for (int m = 0; m < MT16; ++m) {
        __syncthreads();
        float* mine = &sred[warp][0][0];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            mine[g * kDphiCols + 16 * q + u] = acc[m][u][0];
            mine[g * kDphiCols + 16 * q + 8 + u] = acc[m][u][1];
            mine[(g + 8) * kDphiCols + 16 * q + u] = acc[m][u][2];
            mine[(g + 8) * kDphiCols + 16 * q + 8 + u] = acc[m][u][3];
        }
        __syncthreads();
        for (int i = threadIdx.x; i < 16 * kDphiCols; i += kDphiWarps * 32) {
            const int r = row0 + 16 * m + i / kDphiCols, c = i % kDphiCols;
            if (r >= K || col0 + c >= nC) continue;
            float t = 0.f;
#pragma unroll
            for (int wi = 0; wi < kDphiWarps; ++wi) t += (&sred[wi][0][0])[i];
            dphi[(int64_t)r * nC + col0 + c] = t;
        }
    }
}

// Many output rows (wide expansion rates: K = 1088 at n = 32) and few tokens: every warp owns whole
// m16 row tiles of dphi for the block's 64 columns and walks ALL tokens itself, so nothing is
// reduced across warps and each result is stored straight from the accumulators; the block's
// slice of x (64 columns x B tokens) is re-read from L1 by the warps, from HBM once.
__global__ void __launch_bounds__(kDphiWarps * 32)
dphi_rows_mma_kernel(float* __restrict__ dphi, const bf16* __restrict__ x,
                     const bf16* __restrict__ dprT, int64_t B, int64_t Bp, int K, int KP,
                     int64_t nC) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int64_t col0 = (int64_t)blockIdx.x * kDphiCols;
    const bool colin = (col0 + 8 * g) < nC;
    const int64_t ngroups = (B + 15) / 16;
    const int ntile = (KP + 15) / 16;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    const bf16* xcol = x + col0 + 8 * g;
    for (int mt = warp; mt < ntile; mt += kDphiWarps) {
        float acc[8][4];
#pragma unroll
        for (int u = 0; u < 8; ++u)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[u][e] = 0.f;
        const int r0 = 16 * mt + g, r1 = r0 + 8;
        struct Ops {
            uint4 xa, xb, xc, xd;
            uint32_t a0, a1, a2, a3;
        };
        auto fetch = [&](int64_t grp, Ops& o) {
            const int64_t ta = grp * 16 + 2 * q;
            o.xa = zero; o.xb = zero; o.xc = zero; o.xd = zero;
            if (colin) {
                if (ta < B) o.xa = *reinterpret_cast<const uint4*>(xcol + ta * nC);
                if (ta + 1 < B) o.xb = *reinterpret_cast<const uint4*>(xcol + (ta + 1) * nC);
                if (ta + 8 < B) o.xc = *reinterpret_cast<const uint4*>(xcol + (ta + 8) * nC);
                if (ta + 9 < B) o.xd = *reinterpret_cast<const uint4*>(xcol + (ta + 9) * nC);
            }
            o.a0 = (r0 < KP) ? ldg_u32(dprT + (int64_t)r0 * Bp + ta) : 0u;
            o.a1 = (r1 < KP) ? ldg_u32(dprT + (int64_t)r1 * Bp + ta) : 0u;
            o.a2 = (r0 < KP) ? ldg_u32(dprT + (int64_t)r0 * Bp + ta + 8) : 0u;
            o.a3 = (r1 < KP) ? ldg_u32(dprT + (int64_t)r1 * Bp + ta + 8) : 0u;
        };
        Ops cur, nxt;
        fetch(0, cur);
        for (int64_t grp = 0; grp < ngroups; ++grp) {
            // the next group's loads are in flight while this group's MMAs run
            const bool more = grp + 1 < ngroups;
            if (more) fetch(grp + 1, nxt);
            const uint32_t wa[4] = {cur.xa.x, cur.xa.y, cur.xa.z, cur.xa.w};
            const uint32_t wb[4] = {cur.xb.x, cur.xb.y, cur.xb.z, cur.xb.w};
            const uint32_t wc[4] = {cur.xc.x, cur.xc.y, cur.xc.z, cur.xc.w};
            const uint32_t wd[4] = {cur.xd.x, cur.xd.y, cur.xd.z, cur.xd.w};
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint32_t b0e = prmt(wa[p], wb[p], 0x5410), b0o = prmt(wa[p], wb[p], 0x7632);
                const uint32_t b1e = prmt(wc[p], wd[p], 0x5410), b1o = prmt(wc[p], wd[p], 0x7632);
                mma_16816(acc[2 * p], cur.a0, cur.a1, cur.a2, cur.a3, b0e, b1e);
                mma_16816(acc[2 * p + 1], cur.a0, cur.a1, cur.a2, cur.a3, b0o, b1o);
            }
            if (more) cur = nxt;
        }
        // same element map as dphi_mma_kernel: acc[u][0..1] -> row r0, columns 16q+u and 16q+8+u;
        // acc[u][2..3] -> row r1
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int64_t ca = col0 + 16 * q + u, cb = ca + 8;
            if (r0 < K) {
                if (ca < nC) dphi[(int64_t)r0 * nC + ca] = acc[u][0];
                if (cb < nC) dphi[(int64_t)r0 * nC + cb] = acc[u][1];
            }
            if (r1 < K) {
                if (ca < nC) dphi[(int64_t)r1 * nC + ca] = acc[u][2];
                if (cb < nC) dphi[(int64_t)r1 * nC + cb] = acc[u][3];
            }
        }
    }
}

}  // namespace

// ---- host side ---------------------------------------------------------------------------------
bool bwd_mma_supported(Dims d) { return d.n == 4 && d.C % 8 == 0; }

int bwd_mma_kp(Dims d) { return (d.K() + 7) / 8 * 8; }
int bwd_mma_record_floats(Dims d) { return (d.n * d.n + 2 * d.n + 3 + 3) / 4 * 4; }

// dprT[k][b] = bf16(dpr[b][k]) for k < K, b < B; zero in the padding rows K..KP-1 and columns B..Bp-1
__global__ void dpr_transpose_kernel(bf16* __restrict__ dprT, const float* __restrict__ dpr,
                                     int64_t B, int64_t Bp, int K, int KP) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (int64_t)KP * Bp) return;
    const int64_t k = i / Bp, b = i % Bp;
    dprT[i] = __float2bfloat16_rn((k < K && b < B) ? dpr[b * K + k] : 0.f);
}

cudaError_t launch_dpr_transpose(bf16* dprT, const float* dpr, Dims d, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    const int K = d.K(), KP = bwd_mma_kp(d);
    const int64_t Bp = (d.B + 15) / 16 * 16;
    const int64_t total = (int64_t)KP * Bp;
    dpr_transpose_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(dprT, dpr, d.B, Bp, K, KP);
    return launched();
}

cudaError_t launch_dphi_mma(float* dphi, const bf16* x, const bf16* dprT, Dims d, cudaStream_t s) {
    const int K = d.K(), KP = bwd_mma_kp(d);
    const int64_t Bp = (d.B + 15) / 16 * 16;
    const int64_t nC = d.nC();
    if (KP > 8 * 32) {   // many rows: one block per 64 columns, row tiles dealt to the warps
        dphi_rows_mma_kernel<<<(unsigned)((nC + kDphiCols - 1) / kDphiCols), kDphiWarps * 32, 0, s>>>(
            dphi, x, dprT, d.B, Bp, K, KP, nC);
        return launched();
    }
    constexpr int MT16 = 2;
    const dim3 grid((unsigned)((nC + kDphiCols - 1) / kDphiCols),
                    (unsigned)((KP + MT16 * 16 - 1) / (MT16 * 16)));
    dphi_mma_kernel<MT16><<<grid, kDphiWarps * 32, 0, s>>>(dphi, x, dprT, d.B, Bp, K, KP, nC);
    return launched();
}

}  // namespace mhc
