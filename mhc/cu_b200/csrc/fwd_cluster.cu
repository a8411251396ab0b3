// Dynamic-H forward in ONE kernel (bf16, n = 4): x is read from HBM once and y written once.
//
// A thread-block CLUSTER of S blocks owns 16 tokens; block r of the cluster owns the column slice
// [r*Cs, (r+1)*Cs) of all four streams and keeps that tile of x in its shared memory (TMA bulk
// copies, one per token and stream, completed on an mbarrier).  The per-token reductions that span
// the whole row go through distributed shared memory:
//   1. each block contracts its tile with its slice of phi on mma.sync (x fragments from shared
//      memory, phi fragments from L2) and leaves partial projections + sum of squares in smem;
//   2. cluster barrier; every block adds the S partials (reading its peers' shared memory), then
//      computes the 16 tokens' coefficients redundantly (RMS scale, sigmoid / 2*sigmoid / exp,
//      Sinkhorn-Knopp, one thread per token) — no second kernel, no global round trip;
//   3. a = sum_i H_pre[i] x[i,:] over the block's columns, partial sum of squares per token,
//      cluster barrier, add the S partials -> rho;
//   4. y[i,:] = sum_j M[i,j] x[j,:] + H_post[i] a / rho * w from the tile still in shared memory.
// Block 0 of the cluster writes the saved per-token tensors.
//
// Takes over the whole of mhc_layer_fwd_dynamic (src/python/bindings.cu:403-481 of the
// reference: compute_rms, cuBLASLt GEMM, fused_h_activations, batched Sinkhorn, aggregate,
// RMSNorm, distribute+mix — nine launches there).
#include <cooperative_groups.h>

#include "async.cuh"
#include "kernels.h"
#include "sinkhorn.cuh"

namespace cg = cooperative_groups;

namespace mhc {

namespace {

constexpr int kCN = 4;            // streams
constexpr int kCK = 24;           // projection outputs
constexpr int kCTok = 16;         // tokens per cluster
constexpr int kCThreads = 256;
constexpr int kCWarps = 8;
constexpr int kCPart = kCK + 1;   // partial row: 24 projections + sum of squares

__device__ __forceinline__ void c_mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                            uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ float c_sumsq8(const uint4& v) {
    float s = 0.f, t;
    t = bf16_lo(v.x); s = fmaf(t, t, s); t = bf16_hi(v.x); s = fmaf(t, t, s);
    t = bf16_lo(v.y); s = fmaf(t, t, s); t = bf16_hi(v.y); s = fmaf(t, t, s);
    t = bf16_lo(v.z); s = fmaf(t, t, s); t = bf16_hi(v.z); s = fmaf(t, t, s);
    t = bf16_lo(v.w); s = fmaf(t, t, s); t = bf16_hi(v.w); s = fmaf(t, t, s);
    return s;
}

struct ClusterFwdParams {
    bf16* y;
    float* rho;
    float* rms_h;
    float* H_pre;
    float* H_post;
    float* M;
    float* proj;
    float* sk_den;       // may be NULL
    const bf16* x;
    const bf16* w;
    const bf16* phi;     // [24][4C]
    const float* alpha;
    const float* bias;
    int* status;
    int64_t B;
    int64_t C;
    int Cs;              // columns per block = C / cluster size
    int iters;
    float eps;
};

// shared memory (bytes), all offsets multiples of 16:
//   tile   [16][TP]            TP = 4*Cs*2 + 16 (padded token pitch)
//   part   [16][25]            this block's partial (read by the peers)
//   tot    [16][25]            cluster totals
//   coef   [16][28]            MT... layout: hp[4] hq[4] m[16] ri rho_inv pad
//   ssp    [16]                this block's partial sum of a^2 (read by the peers)
//   bar    mbarrier
constexpr int kCoefF = 28;   // 16 * 28 >= 16 * 25: coef doubles as a scratch tile of the cross-warp sum

__global__ void __launch_bounds__(kCThreads, 3)
fwd_cluster_kernel(const ClusterFwdParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    cg::cluster_group cluster = cg::this_cluster();
    const int S = (int)cluster.num_blocks();
    const int rank = (int)cluster.block_rank();
    const int Cs = p.Cs;
    const int64_t C = p.C, nC = 4 * C;
    const int TP = kCN * Cs * 2 + 16;
    unsigned char* tile = smem;
    float* part = reinterpret_cast<float*>(smem + kCTok * TP);
    float* tot = part + kCTok * kCPart;
    float* coef = tot + kCTok * kCPart;
    float* ssp = coef + kCTok * kCoefF;
    uint64_t* bar = reinterpret_cast<uint64_t*>(ssp + kCTok);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, q = lane & 3;
    const int64_t t0 = (int64_t)blockIdx.y * kCTok;
    int nvalid = (int)((p.B - t0 < kCTok) ? (p.B - t0) : kCTok);
    const int64_t col0 = (int64_t)rank * Cs;        // first column of this block's slice

    // ---- 1. stage the tile: one bulk copy per (token, stream) ---------------------------------
    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init_fence();
        mbar_arrive_expect_tx(bar, (uint32_t)(nvalid * kCN * Cs * 2));
    }
    __syncthreads();
    if (tid < kCTok * kCN) {
        const int t = tid >> 2, j = tid & 3;
        if (t < nvalid)
            bulk_copy_g2s(tile + t * TP + j * Cs * 2, p.x + (t0 + t) * nC + (int64_t)j * C + col0,
                          (uint32_t)(Cs * 2), bar);
    }

    // ---- 2. contraction of the tile with this block's slice of phi -------------------------------
    // chunks of 32 flat elements; chunk c lies in stream c / (Cs/32) at column (c % (Cs/32)) * 32
    const int cps = Cs / 32;                 // chunks per stream
    const int nchunk = kCN * cps;
    float acc[3][4];
#pragma unroll
    for (int t = 0; t < 3; ++t)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
    float sslo = 0.f, sshi = 0.f;
    const bf16* prow[3];
#pragma unroll
    for (int t = 0; t < 3; ++t) prow[t] = p.phi + (int64_t)(8 * t + g) * nC;

    // phi fragments of up to four chunks are requested first (they do not depend on x), then the
    // block waits once for the tile; the vote keeps the decision uniform over the block
    uint4 pf[4][3];
    auto load_phi = [&](int cb) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = cb + u * kCWarps;
            if (c < nchunk) {
                const int64_t off = (int64_t)(c / cps) * C + col0 + (c % cps) * 32 + 8 * q;
#pragma unroll
                for (int t = 0; t < 3; ++t)
                    pf[u][t] = *reinterpret_cast<const uint4*>(prow[t] + off);
            }
        }
    };
    load_phi(warp);
    {
        const int ok = __syncthreads_and(mbar_wait_bounded(bar, 0) ? 1 : 0);
        if (!ok) {
            if (tid == 0 && p.status != nullptr) atomicOr(p.status, kDevErrBulkWait);
            // the peers wait at the cluster barriers below: keep the protocol, skip the work
            cluster.sync();
            cluster.sync();
            cluster.sync();
            return;
        }
    }
    for (int cb = warp; cb < nchunk; cb += 4 * kCWarps) {
        if (cb != warp) load_phi(cb);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int c = cb + u * kCWarps;
            if (c < nchunk) {
                const int boff = (c / cps) * Cs * 2 + ((c % cps) * 32 + 8 * q) * 2;
                const uint4 r = *reinterpret_cast<const uint4*>(tile + g * TP + boff);
                const uint4 s = *reinterpret_cast<const uint4*>(tile + (g + 8) * TP + boff);
#pragma unroll
                for (int t = 0; t < 3; ++t) {
                    c_mma_16816(acc[t], r.x, s.x, r.y, s.y, pf[u][t].x, pf[u][t].y);
                    c_mma_16816(acc[t], r.z, s.z, r.w, s.w, pf[u][t].z, pf[u][t].w);
                }
                sslo += c_sumsq8(r);
                sshi += c_sumsq8(s);
            }
        }
    }
    // cross-warp sum in a fixed order with three scratch tiles (part, tot, coef are free until the
    // cluster totals): warps 0-2 store, warps 3-5 add, warps 6-7 add, then the three tiles are added
    sslo += __shfl_xor_sync(0xffffffffu, sslo, 1);
    sslo += __shfl_xor_sync(0xffffffffu, sslo, 2);
    sshi += __shfl_xor_sync(0xffffffffu, sshi, 1);
    sshi += __shfl_xor_sync(0xffffffffu, sshi, 2);
#pragma unroll
    for (int round = 0; round < 3; ++round) {
        if (warp / 3 == round) {
            float* dst = (warp % 3 == 0) ? part : (warp % 3 == 1) ? tot : coef;
#pragma unroll
            for (int t = 0; t < 3; ++t) {
                float* lo = dst + g * kCPart + 8 * t + 2 * q;
                float* hi = dst + (g + 8) * kCPart + 8 * t + 2 * q;
                lo[0] = (round == 0 ? 0.f : lo[0]) + acc[t][0];
                lo[1] = (round == 0 ? 0.f : lo[1]) + acc[t][1];
                hi[0] = (round == 0 ? 0.f : hi[0]) + acc[t][2];
                hi[1] = (round == 0 ? 0.f : hi[1]) + acc[t][3];
            }
            if (q == 0) {
                float* lo = dst + g * kCPart + kCK;
                float* hi = dst + (g + 8) * kCPart + kCK;
                lo[0] = (round == 0 ? 0.f : lo[0]) + sslo;
                hi[0] = (round == 0 ? 0.f : hi[0]) + sshi;
            }
        }
        __syncthreads();
    }
    for (int i = tid; i < kCTok * kCPart; i += kCThreads) part[i] = (part[i] + tot[i]) + coef[i];
    cluster.sync();   // (1) every block's partial is in place

    // ---- 3. cluster totals, then the 16 tokens' coefficients (redundantly in every block) ----------
    for (int i = tid; i < kCTok * kCPart; i += kCThreads) {
        float v = 0.f;
        for (int r = 0; r < S; ++r) v += cluster.map_shared_rank(part, r)[i];
        tot[i] = v;
    }
    __syncthreads();
    // activations: item = (token, k)
    for (int i = tid; i < kCTok * kCK; i += kCThreads) {
        const int t = i / kCK, k = i % kCK;
        const float r = sqrtf(tot[t * kCPart + kCK] / (float)nC + p.eps);
        const float pv = tot[t * kCPart + k] / r;
        float* cf = coef + t * kCoefF;
        if (rank == 0 && t < nvalid) {
            p.proj[(t0 + t) * kCK + k] = pv;
            if (k == 0) p.rms_h[t0 + t] = r;
        }
        if (k < 4) {
            const float h = sk_sigmoid<float>(p.alpha[0] * pv + p.bias[k]);
            cf[k] = h;
            if (rank == 0 && t < nvalid) p.H_pre[(t0 + t) * 4 + k] = h;
        } else if (k < 8) {
            const float h = 2.f * sk_sigmoid<float>(p.alpha[1] * pv + p.bias[k]);
            cf[k] = h;
            if (rank == 0 && t < nvalid) p.H_post[(t0 + t) * 4 + (k - 4)] = h;
        } else {
            cf[k] = expf(p.alpha[2] * pv + p.bias[k]);     // E, row major at cf[8 .. 24)
        }
    }
    __syncthreads();
    if (tid < kCTok) {
        float* cf = coef + tid * kCoefF;
        float m[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) m[i][j] = cf[8 + i * 4 + j];
        const bool keep = rank == 0 && tid < nvalid && p.sk_den != nullptr;
        if (keep)
            sk_forward_thread<4, float, true>(m, 4, p.iters, p.eps,
                                              p.sk_den + (t0 + tid) * 2 * (int64_t)p.iters * 4);
        else
            sk_forward_thread<4, float, false>(m, 4, p.iters, p.eps, nullptr);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                cf[8 + i * 4 + j] = m[i][j];
                if (rank == 0 && tid < nvalid) p.M[(t0 + tid) * 16 + i * 4 + j] = m[i][j];
            }
    }
    __syncthreads();

    // ---- 4. pass 1 over the tile: partial sum of squares of the aggregated stream --------------
    // warp w handles tokens 2w and 2w+1; lanes stride over the 8-column vectors of the slice
    const int nvec = Cs / 8;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int t = 2 * warp + h;
        const float* cf = coef + t * kCoefF;
        const float hp0 = cf[0], hp1 = cf[1], hp2 = cf[2], hp3 = cf[3];
        float ss = 0.f;
        for (int v = lane; v < nvec; v += 32) {
            float a[8], xv[8];
            load_vec<8>(reinterpret_cast<const bf16*>(tile + t * TP) + v * 8, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = hp0 * xv[e];
            load_vec<8>(reinterpret_cast<const bf16*>(tile + t * TP + Cs * 2) + v * 8, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = fmaf(hp1, xv[e], a[e]);
            load_vec<8>(reinterpret_cast<const bf16*>(tile + t * TP + 2 * Cs * 2) + v * 8, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) a[e] = fmaf(hp2, xv[e], a[e]);
            load_vec<8>(reinterpret_cast<const bf16*>(tile + t * TP + 3 * Cs * 2) + v * 8, xv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                a[e] = fmaf(hp3, xv[e], a[e]);
                ss = fmaf(a[e], a[e], ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) ssp[t] = ss;
    }
    cluster.sync();   // (2) every block's partial sums of squares are in place
    if (tid < kCTok) {
        float v = 0.f;
        for (int r = 0; r < S; ++r) v += cluster.map_shared_rank(ssp, r)[tid];
        const float rho = sqrtf(v / (float)C + p.eps);
        coef[tid * kCoefF + 24] = 1.f / rho;
        if (rank == 0 && tid < nvalid) p.rho[t0 + tid] = rho;
    }
    cluster.sync();   // (3) nobody reads a peer's shared memory after this point

    // ---- 5. pass 2: the outputs of this block's columns ------------------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int t = 2 * warp + h;
        if (t >= nvalid) continue;
        const float* cf = coef + t * kCoefF;
        float hp[4], hq[4], m[4][4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            hp[i] = cf[i];
            hq[i] = cf[4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) m[i][j] = cf[8 + i * 4 + j];
        }
        const float ri = cf[24];
        bf16* yb = p.y + (t0 + t) * nC + col0;
        for (int v = lane; v < nvec; v += 32) {
            float xv[4][8], wv[8], yn[8];
#pragma unroll
            for (int i = 0; i < 4; ++i)
                load_vec<8>(reinterpret_cast<const bf16*>(tile + t * TP + i * Cs * 2) + v * 8, xv[i]);
            load_weight<8>(p.w, col0 + v * 8, wv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float a = hp[0] * xv[0][e];
                a = fmaf(hp[1], xv[1][e], a);
                a = fmaf(hp[2], xv[2][e], a);
                a = fmaf(hp[3], xv[3][e], a);
                yn[e] = a * ri * wv[e];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float o[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float tt = hq[i] * yn[e];
#pragma unroll
                    for (int j = 0; j < 4; ++j) tt = fmaf(m[i][j], xv[j][e], tt);
                    o[e] = tt;
                }
                store_vec<8>(yb + (int64_t)i * C + v * 8, o);
            }
        }
    }
}

size_t cluster_smem(int Cs) {
    const size_t tile = (size_t)kCTok * (kCN * Cs * 2 + 16);
    const size_t floats = (size_t)2 * kCTok * kCPart + kCTok * kCoefF + kCTok;
    return tile + floats * 4 + 16;
}

}  // namespace

// Cluster size for this shape, 0 if the fused forward does not cover it: n = 4, bf16, the column
// slice of a block a multiple of 32 columns and at most 512 columns wide.
int fwd_cluster_size(Dims d) {
    if (d.n != 4 || d.B == 0) return 0;
    for (int S = 1; S <= 8; ++S) {
        if (d.C % (32 * S) != 0) continue;
        const int64_t Cs = d.C / S;
        if (Cs <= 512) return S;
    }
    return 0;
}

cudaError_t launch_fwd_cluster(bf16* y, float* rho, float* rms_h, float* H_pre, float* H_post,
                               float* M, float* proj, float* sk_den, const bf16* x, const bf16* w,
                               const bf16* phi, const float* alpha, const float* bias, int* status,
                               Dims d, int iters, float eps, cudaStream_t s) {
    const int S = fwd_cluster_size(d);
    if (S == 0) return cudaErrorNotSupported;
    ClusterFwdParams p{y, rho, rms_h, H_pre, H_post, M, proj, sk_den, x, w, phi, alpha, bias, status,
                       d.B, d.C, (int)(d.C / S), iters, eps};
    const size_t smem = cluster_smem(p.Cs);
    cudaError_t e = cudaFuncSetAttribute(fwd_cluster_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)S, (unsigned)((d.B + kCTok - 1) / kCTok), 1);
    cfg.blockDim = dim3(kCThreads, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, fwd_cluster_kernel, p);
    if (e != cudaSuccess) return e;
    return launched();
}

}  // namespace mhc
