// bf16 projection on the tensor cores:  praw[b,k] = sum_m x_flat[b,m] * phi[k,m],  sumsq[b] = |x_b|^2.
//
// This is a GEMM with a tiny N (K = 2n + n^2 = 24 outputs at n = 4) and a long reduction
// (nC = 10240): HBM-bound on reading x once, but 24 FMA per loaded element is more than the
// fp32 pipes deliver at that rate, so the products go through mma.sync.m16n8k16 (bf16 in, fp32
// accumulate).  x is the A operand (16 tokens per warp), phi the B operand (8 outputs per tile).
//
// No shared-memory staging of the operands is needed: the reduction index may be permuted freely
// as long as A and B use the same permutation, so every thread loads 16 contiguous bytes of its
// token row (and of its phi row) and feeds the four 32-bit words straight into two MMAs.
//
// Work split: block = 8 warps that share 16 tokens and one slice of the reduction axis, each warp
// taking an eighth of the slice; their partial tiles are added in shared memory and the block
// writes one partial result  praw_part[slice][b][k]  (summed later by the coefficient kernel, in
// a fixed order).
//
// Takes over compute_rms + the cuBLASLt bf16 GEMM of the reference
// (src/csrc/kernels/fused_rmsnorm_matmul.cuh:15-153, src/python/bindings.cu:21-111,426-443).
#include "kernels.h"

namespace mhc {

namespace {

constexpr int kWarps = 8;
constexpr int kTokens = 16;   // tokens per block (the M of m16n8k16)
constexpr int kChunk = 32;    // reduction elements per warp step (two k16 MMAs)

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                               uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float sumsq8(const uint4& v) {
    float s = 0.f, t;
    t = bf16_lo(v.x); s = fmaf(t, t, s); t = bf16_hi(v.x); s = fmaf(t, t, s);
    t = bf16_lo(v.y); s = fmaf(t, t, s); t = bf16_hi(v.y); s = fmaf(t, t, s);
    t = bf16_lo(v.z); s = fmaf(t, t, s); t = bf16_hi(v.z); s = fmaf(t, t, s);
    t = bf16_lo(v.w); s = fmaf(t, t, s); t = bf16_hi(v.w); s = fmaf(t, t, s);
    return s;
}

// NT = output tiles of 8 handled by one block (blockIdx.z picks the group of NT tiles).
// CH = chunks of 32 reduction elements per warp (compile-time so that all loads of x are issued
// before the first MMA).
template <int NT, int CH>
__global__ void __launch_bounds__(kWarps * 32, (NT * CH <= 15) ? 2 : 1)
proj_mma_kernel(float* __restrict__ praw_part, float* __restrict__ sumsq_part,
                const bf16* __restrict__ x, const bf16* __restrict__ phi, int64_t B, int K,
                int64_t nC) {
    constexpr int NOUT = NT * 8;
    __shared__ float red[kWarps][kTokens][NOUT + 1];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int64_t t0 = (int64_t)blockIdx.x * kTokens;
    const int64_t slice = (int64_t)kWarps * CH * kChunk;          // reduction elements per block
    const int64_t kbeg = (int64_t)blockIdx.y * slice + (int64_t)warp * CH * kChunk;
    const int out0 = blockIdx.z * NOUT;

    const int64_t tlo = t0 + g, thi = t0 + g + 8;
    const bool vlo = tlo < B, vhi = thi < B;
    const bf16* xlo = x + (vlo ? tlo : 0) * nC;
    const bf16* xhi = x + (vhi ? thi : 0) * nC;

    uint4 r[CH], s[CH];
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int64_t k = kbeg + (int64_t)c * kChunk + 8 * q;
        const bool in = k < nC;  // nC is a multiple of 8, so a started vector is a whole vector
        r[c] = (in && vlo) ? *reinterpret_cast<const uint4*>(xlo + k) : zero;
        s[c] = (in && vhi) ? *reinterpret_cast<const uint4*>(xhi + k) : zero;
    }

    float acc[NT][4];
#pragma unroll
    for (int t = 0; t < NT; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;

    const bf16* prow[NT];
    bool pval[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        const int row = out0 + 8 * t + g;
        pval[t] = row < K;
        prow[t] = phi + (int64_t)(pval[t] ? row : 0) * nC;
    }

    // all phi fragments of this warp's slice are requested before the first MMA, so x (HBM) and
    // phi (L2) arrive within one round trip instead of one per chunk
    uint4 pf[CH][NT];
#pragma unroll
    for (int c = 0; c < CH; ++c) {
        const int64_t k = kbeg + (int64_t)c * kChunk + 8 * q;
        const bool in = k < nC;
#pragma unroll
        for (int t = 0; t < NT; ++t)
            pf[c][t] = (in && pval[t]) ? *reinterpret_cast<const uint4*>(prow[t] + k) : zero;
    }
    float sslo = 0.f, sshi = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const uint4 p = pf[c][t];
            mma_bf16_16816(acc[t], r[c].x, s[c].x, r[c].y, s[c].y, p.x, p.y);
            mma_bf16_16816(acc[t], r[c].z, s[c].z, r[c].w, s[c].w, p.z, p.w);
        }
        if (blockIdx.z == 0) {
            sslo += sumsq8(r[c]);
            sshi += sumsq8(s[c]);
        }
    }
    // accumulator layout: acc[t][0..1] -> (token g, outputs 8t+2q, +1); acc[t][2..3] -> token g+8
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        red[warp][g][8 * t + 2 * q] = acc[t][0];
        red[warp][g][8 * t + 2 * q + 1] = acc[t][1];
        red[warp][g + 8][8 * t + 2 * q] = acc[t][2];
        red[warp][g + 8][8 * t + 2 * q + 1] = acc[t][3];
    }
    sslo += __shfl_xor_sync(0xffffffffu, sslo, 1);
    sslo += __shfl_xor_sync(0xffffffffu, sslo, 2);
    sshi += __shfl_xor_sync(0xffffffffu, sshi, 1);
    sshi += __shfl_xor_sync(0xffffffffu, sshi, 2);
    if (q == 0) {
        red[warp][g][NOUT] = sslo;
        red[warp][g + 8][NOUT] = sshi;
    }
    __syncthreads();
    const int64_t part = blockIdx.y;
    for (int i = threadIdx.x; i < kTokens * (NOUT + 1); i += kWarps * 32) {
        const int tok = i / (NOUT + 1), o = i % (NOUT + 1);
        if (t0 + tok >= B) continue;
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) v += red[w][tok][o];
        if (o < NOUT) {
            if (out0 + o < K) praw_part[(part * B + t0 + tok) * K + out0 + o] = v;
        } else if (blockIdx.z == 0) {
            sumsq_part[part * B + t0 + tok] = v;
        }
    }
}

}  // namespace

// Number of partial results the kernel produces for this shape (0: shape not covered).
int proj_mma_splits(Dims d) {
    if (d.nC() % 8 != 0) return 0;
    const int64_t per_block_ch1 = (int64_t)kWarps * kChunk;  // 256 reduction elements with CH = 1
    // aim for about four blocks per SM over the token groups
    const int64_t groups = (d.B + kTokens - 1) / kTokens;
    int64_t want = (4 * 148 + groups - 1) / groups;
    if (want < 1) want = 1;
    int64_t ch = (d.nC() + want * per_block_ch1 - 1) / (want * per_block_ch1);
    if (ch < 1) ch = 1;
    if (ch > 8) ch = 8;
    // round to a compiled chunk count
    const int compiled[] = {1, 2, 3, 4, 5, 6, 8};
    int pick = 8;
    for (int c : compiled)
        if (c >= ch) { pick = c; break; }
    const int64_t slice = per_block_ch1 * pick;
    return (int)((d.nC() + slice - 1) / slice) | (pick << 24);
}

template <int NT>
static cudaError_t proj_mma_launch(float* praw_part, float* sumsq_part, const bf16* x,
                                   const bf16* phi, Dims d, int splits, int ch, int zgroups,
                                   cudaStream_t s) {
    const dim3 grid((unsigned)((d.B + kTokens - 1) / kTokens), (unsigned)splits, (unsigned)zgroups);
    const int K = d.K();
#define MHC_PM(CH_)                                                                           \
    case CH_:                                                                                 \
        proj_mma_kernel<NT, CH_><<<grid, kWarps * 32, 0, s>>>(praw_part, sumsq_part, x, phi, d.B, \
                                                              K, d.nC());                     \
        break;
    switch (ch) {
        MHC_PM(1) MHC_PM(2) MHC_PM(3) MHC_PM(4) MHC_PM(5) MHC_PM(6) MHC_PM(8)
        default: return cudaErrorInvalidValue;
    }
#undef MHC_PM
    return launched();
}

cudaError_t launch_proj_mma(float* praw_part, float* sumsq_part, const bf16* x, const bf16* phi,
                            Dims d, cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    const int packed = proj_mma_splits(d);
    if (packed == 0) return cudaErrorNotSupported;
    const int splits = packed & 0xffffff, ch = packed >> 24;
    const int tiles = (d.K() + 7) / 8;
    if (tiles <= 1) return proj_mma_launch<1>(praw_part, sumsq_part, x, phi, d, splits, ch, 1, s);
    if (tiles == 2) return proj_mma_launch<2>(praw_part, sumsq_part, x, phi, d, splits, ch, 1, s);
    if (tiles == 3) return proj_mma_launch<3>(praw_part, sumsq_part, x, phi, d, splits, ch, 1, s);
    if (tiles == 4) return proj_mma_launch<4>(praw_part, sumsq_part, x, phi, d, splits, ch, 1, s);
    return proj_mma_launch<5>(praw_part, sumsq_part, x, phi, d, splits, ch, (tiles + 4) / 5, s);
}

}  // namespace mhc
