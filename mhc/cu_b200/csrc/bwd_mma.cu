// bf16 backward passes that contain a contraction against phi, on mma.sync tensor-core tiles:
//
//   dx_mma    dx[b,j,c] = sum_i M[i,j] g[i,c] + H_pre[j] da[c] - qq x[j,c] + sum_k dpr[b,k] phi[k, jC+c]
//             The last term is a [tokens x K] x [K x columns] product (K = 2n + n^2 = 24 at n = 4):
//             A = dpr (16 tokens), B = phi fragments kept in shared memory, accumulators land
//             exactly on the (token, 8 contiguous columns) patch the same thread then finishes
//             element-wise, so x, dy are read once and dx is written once.
//   dphi_mma  dphi[k,m] = sum_b dpr[b,k] x[b,m]: A = dpr^T, B = x with token pairs interleaved in
//             registers (PRMT), one block owns 64 columns for all tokens, so dphi is written once,
//             in a fixed summation order.
//
// Both read small bf16 copies of dpr that the coefficient kernel writes: dprb[B][KP] (token major)
// and dprT[KP][Bp] (k major), KP = K rounded up to 8, Bp = B rounded up to 16.
//
// Takes over the eager GEMMs d_x_flat = d_p @ phi and d_phi = d_p^T @ x_flat of the reference's
// dynamic backward (src/python/mhc/ops.py:330-349) and its stream_distribute_mix_backward /
// stream_aggregate_backward / rmsnorm_backward kernels (src/csrc/kernels/stream_ops.cuh:644-997,
// src/csrc/kernels/rmsnorm.cuh:233-306).
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
__device__ __forceinline__ void mma_1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, "
        "{%0,%1,%2,%3};\n"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(b0));
}

// 16-byte asynchronous copy global -> shared (Ampere-style cp.async, lands without occupying
// registers); src_bytes = 0 writes zeros instead of reading.
__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(dst_smem)),
                 "l"(src), "r"(src_bytes)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ uint32_t ldg_u32(const bf16* p) {
    return *reinterpret_cast<const uint32_t*>(p);
}

// ------------------------------------------------------------------------------------------------
// dx.  N = streams (compile time).  Block = 4 warps, one 32-column block (of every stream), a
// contiguous range of token groups (16 tokens each) dealt round-robin to the warps.
// Thread (g = lane/4, q = lane%4) owns tokens {g, g+8} of its group and columns [8q, 8q+8).
template <int N>
struct DxCfg {
    static constexpr int K = 2 * N + N * N;
    static constexpr int KP = (K + 7) / 8 * 8;    // padded contraction length
    static constexpr int K16 = KP / 16;            // k16 MMA steps
    static constexpr int K8 = (KP % 16) ? 1 : 0;   // plus one k8 step
    static constexpr int FW = 2 * K16 + K8;        // 32-bit words of B fragment per (stream, tile)
    static constexpr int FWP = (FW + 3) / 4 * 4;   // padded to 16-byte loads
    static constexpr int RS = (N * N + 2 * N + 3 + 3) / 4 * 4;  // floats per token record
};

constexpr int kDxWarps = 4;
constexpr int kDxCols = 32;

// Per-token record written by the coefficient kernel (fp32):
//   [0, N*N)        MT[j][i] = M[i][j]           (column j of M contiguous)
//   [N*N, +N)       H_pre
//   [N*N+N, +N)     H_post
//   then c1 = 1/rho, c2 = s/(C rho^3), qq.
template <int N>
__global__ void __launch_bounds__(kDxWarps * 32, 3)
dx_mma_kernel(bf16* __restrict__ dx, float* __restrict__ dw_part, const bf16* __restrict__ x,
              const bf16* __restrict__ gy, const bf16* __restrict__ w,
              const float* __restrict__ rec, const bf16* __restrict__ dprb,
              const bf16* __restrict__ phi, int64_t B, int64_t C, int groups_per_block) {
    using Cfg = DxCfg<N>;
    constexpr int K = Cfg::K, KP = Cfg::KP, K16 = Cfg::K16, K8 = Cfg::K8, FWP = Cfg::FWP,
                  RS = Cfg::RS;
    __shared__ __align__(16) uint32_t fragB[N][4][32][FWP];
    __shared__ float dws[kDxWarps][kDxCols];
    // per-thread landing slots of the x / dy patches, double buffered: [buf][vector][thread]
    extern __shared__ __align__(16) uint4 patch[];
    constexpr int NV = 4 * N;   // vectors per patch: {x, dy} x 2 tokens x N streams

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, q = lane & 3;
    const int64_t c0 = (int64_t)blockIdx.x * kDxCols;   // first column of the block
    const int64_t nC = (int64_t)N * C;

    // ---- stage the phi fragments of this column block -----------------------------------------
    // tile t, lane (g,q) supplies column  c0 + 8*(g/2) + 2t + (g%2)  of stream j.
    for (int e = threadIdx.x; e < N * 4 * 32; e += kDxWarps * 32) {
        const int l = e & 31, t = (e >> 5) & 3, j = e >> 7;
        const int lg = l >> 2, lq = l & 3;
        const int64_t col = (int64_t)j * C + c0 + 8 * (lg >> 1) + 2 * t + (lg & 1);
        const bool cin = (c0 + 8 * (lg >> 1) + 2 * t + (lg & 1)) < C;
        auto pair = [&](int k) -> uint32_t {   // (phi[k][col], phi[k+1][col]) as bf16x2
            uint32_t lo = 0, hi = 0;
            if (cin && k < K) lo = *reinterpret_cast<const uint16_t*>(phi + (int64_t)k * nC + col);
            if (cin && k + 1 < K)
                hi = *reinterpret_cast<const uint16_t*>(phi + (int64_t)(k + 1) * nC + col);
            return lo | (hi << 16);
        };
#pragma unroll
        for (int s = 0; s < K16; ++s) {
            fragB[j][t][l][2 * s] = pair(16 * s + 2 * lq);
            fragB[j][t][l][2 * s + 1] = pair(16 * s + 2 * lq + 8);
        }
        if (K8) fragB[j][t][l][2 * K16] = pair(16 * K16 + 2 * lq);
    }
    __syncthreads();

    float wv[8];
    {
        const int64_t c = c0 + 8 * q;
        if (c < C) {
            load_weight<8>(w, c, wv);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) wv[e] = 0.f;
        }
    }
    float dwacc[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) dwacc[e] = 0.f;

    const int64_t group0 = (int64_t)blockIdx.y * groups_per_block;
    const int64_t ngroups = (B + 15) / 16;
    const bool colin = (c0 + 8 * q) < C;   // C is a multiple of 8: whole vector in or out

    // issue the asynchronous loads of one token group's patches into buffer `buf`
    auto prefetch = [&](int64_t grp, int buf) {
        uint4* slot = patch + (size_t)buf * NV * (kDxWarps * 32) + threadIdx.x;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int64_t t = grp * 16 + g + 8 * h;
            const bool ld = (t < B) && colin;
            const int64_t base = (ld ? t : 0) * nC + (colin ? c0 + 8 * q : 0);
#pragma unroll
            for (int i = 0; i < N; ++i) {
                cp_async16(slot + (size_t)((h * N + i) * 2 + 0) * (kDxWarps * 32), x + base + i * C,
                           ld ? 16u : 0u);
                cp_async16(slot + (size_t)((h * N + i) * 2 + 1) * (kDxWarps * 32), gy + base + i * C,
                           ld ? 16u : 0u);
            }
        }
        cp_async_commit();
    };

    int buf = 0;
    if (group0 + warp < ngroups && warp < groups_per_block) prefetch(group0 + warp, 0);
    for (int gi = warp; gi < groups_per_block; gi += kDxWarps) {
        const int64_t grp = group0 + gi;
        if (grp >= ngroups) break;
        const int64_t tok[2] = {grp * 16 + g, grp * 16 + g + 8};
        const bool tv[2] = {tok[0] < B, tok[1] < B};
        const bool more = (gi + kDxWarps < groups_per_block) && (grp + kDxWarps < ngroups);
        if (more) prefetch(grp + kDxWarps, buf ^ 1);

        // A fragments of dpr for this token group
        uint32_t a[K16][4], a8[2] = {0u, 0u};
        {
            const bf16* d0 = dprb + (tv[0] ? tok[0] : 0) * KP;
            const bf16* d1 = dprb + (tv[1] ? tok[1] : 0) * KP;
#pragma unroll
            for (int s = 0; s < K16; ++s) {
                a[s][0] = tv[0] ? ldg_u32(d0 + 16 * s + 2 * q) : 0u;
                a[s][1] = tv[1] ? ldg_u32(d1 + 16 * s + 2 * q) : 0u;
                a[s][2] = tv[0] ? ldg_u32(d0 + 16 * s + 2 * q + 8) : 0u;
                a[s][3] = tv[1] ? ldg_u32(d1 + 16 * s + 2 * q + 8) : 0u;
            }
            if (K8) {
                a8[0] = tv[0] ? ldg_u32(d0 + 16 * K16 + 2 * q) : 0u;
                a8[1] = tv[1] ? ldg_u32(d1 + 16 * K16 + 2 * q) : 0u;
            }
        }

        // this thread's patch of x and dy (2 tokens x N streams x 8 columns, packed bf16) has
        // landed in its own slots once all but the newest copy group are complete
        if (more) cp_async_wait<1>(); else cp_async_wait<0>();
        uint4 xp[2][N], gp[2][N];
        {
            const uint4* slot = patch + (size_t)buf * NV * (kDxWarps * 32) + threadIdx.x;
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    xp[h][i] = slot[(size_t)((h * N + i) * 2 + 0) * (kDxWarps * 32)];
                    gp[h][i] = slot[(size_t)((h * N + i) * 2 + 1) * (kDxWarps * 32)];
                }
        }
        buf ^= 1;

        // da and the d_weight contribution per token
        float da[2][8];
        float qq[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const float* r = rec + (tv[h] ? tok[h] : 0) * RS;
            float hp[N], hq[N];
#pragma unroll
            for (int i = 0; i < N; ++i) {
                hp[i] = r[N * N + i];
                hq[i] = r[N * N + N + i];
            }
            const float c1 = r[N * N + 2 * N], c2 = r[N * N + 2 * N + 1];
            qq[h] = r[N * N + 2 * N + 2];
            float av[8], dv[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) { av[e] = 0.f; dv[e] = 0.f; }
#pragma unroll
            for (int i = 0; i < N; ++i) {
                const uint32_t xw[4] = {xp[h][i].x, xp[h][i].y, xp[h][i].z, xp[h][i].w};
                const uint32_t gw[4] = {gp[h][i].x, gp[h][i].y, gp[h][i].z, gp[h][i].w};
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    av[2 * p] = fmaf(hp[i], bf16_lo(xw[p]), av[2 * p]);
                    av[2 * p + 1] = fmaf(hp[i], bf16_hi(xw[p]), av[2 * p + 1]);
                    dv[2 * p] = fmaf(hq[i], bf16_lo(gw[p]), dv[2 * p]);
                    dv[2 * p + 1] = fmaf(hq[i], bf16_hi(gw[p]), dv[2 * p + 1]);
                }
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                da[h][e] = dv[e] * wv[e] * c1 - av[e] * c2;
                if (tv[h]) dwacc[e] = fmaf(dv[e] * c1, av[e], dwacc[e]);
            }
        }

        // stream by stream: tensor-core term, then the element-wise rest, then store
#pragma unroll
        for (int j = 0; j < N; ++j) {
            float acc[4][4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[t][e] = 0.f;
                uint32_t fb[FWP];
                if constexpr (FWP == 4) {
                    const uint4 v = *reinterpret_cast<const uint4*>(&fragB[j][t][lane][0]);
                    fb[0] = v.x; fb[1] = v.y; fb[2] = v.z; fb[3] = v.w;
                } else {
#pragma unroll
                    for (int u = 0; u < FWP; u += 4) {
                        const uint4 v = *reinterpret_cast<const uint4*>(&fragB[j][t][lane][u]);
                        fb[u] = v.x; fb[u + 1] = v.y; fb[u + 2] = v.z; fb[u + 3] = v.w;
                    }
                }
#pragma unroll
                for (int s = 0; s < K16; ++s)
                    mma_16816(acc[t], a[s][0], a[s][1], a[s][2], a[s][3], fb[2 * s], fb[2 * s + 1]);
                if (K8) mma_1688(acc[t], a8[0], a8[1], fb[2 * K16]);
            }
            // acc[t][e] -> (token g, column 8q + 2t + e); acc[t][2+e] -> token g+8
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const float* r = rec + (tv[h] ? tok[h] : 0) * RS;
                float mt[N];
#pragma unroll
                for (int i = 0; i < N; ++i) mt[i] = r[j * N + i];
                const float hpj = r[N * N + j];
                float o[8];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    o[2 * t] = acc[t][2 * h];
                    o[2 * t + 1] = acc[t][2 * h + 1];
                }
                const uint32_t xw[4] = {xp[h][j].x, xp[h][j].y, xp[h][j].z, xp[h][j].w};
#pragma unroll
                for (int p = 0; p < 4; ++p) {
                    o[2 * p] = fmaf(-qq[h], bf16_lo(xw[p]), fmaf(hpj, da[h][2 * p], o[2 * p]));
                    o[2 * p + 1] =
                        fmaf(-qq[h], bf16_hi(xw[p]), fmaf(hpj, da[h][2 * p + 1], o[2 * p + 1]));
                }
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    const uint32_t gw[4] = {gp[h][i].x, gp[h][i].y, gp[h][i].z, gp[h][i].w};
#pragma unroll
                    for (int p = 0; p < 4; ++p) {
                        o[2 * p] = fmaf(mt[i], bf16_lo(gw[p]), o[2 * p]);
                        o[2 * p + 1] = fmaf(mt[i], bf16_hi(gw[p]), o[2 * p + 1]);
                    }
                }
                if (tv[h] && colin) {
                    uint4 ov;
                    ov.x = pack_bf16x2(o[0], o[1]);
                    ov.y = pack_bf16x2(o[2], o[3]);
                    ov.z = pack_bf16x2(o[4], o[5]);
                    ov.w = pack_bf16x2(o[6], o[7]);
                    *reinterpret_cast<uint4*>(dx + tok[h] * nC + j * C + c0 + 8 * q) = ov;
                }
            }
        }
    }

    // d_weight partial of this block: sum over the 8 token lanes (g), then over the warps
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        float v = dwacc[e];
        v += __shfl_xor_sync(0xffffffffu, v, 4);
        v += __shfl_xor_sync(0xffffffffu, v, 8);
        v += __shfl_xor_sync(0xffffffffu, v, 16);
        dwacc[e] = v;
    }
    if (g == 0) {
#pragma unroll
        for (int e = 0; e < 8; ++e) dws[warp][8 * q + e] = dwacc[e];
    }
    __syncthreads();
    if (threadIdx.x < kDxCols && c0 + threadIdx.x < C) {
        float t = 0.f;
#pragma unroll
        for (int wi = 0; wi < kDxWarps; ++wi) t += dws[wi][threadIdx.x];
        dw_part[(int64_t)blockIdx.y * C + c0 + threadIdx.x] = t;
    }
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

}  // namespace

// ---- host side ---------------------------------------------------------------------------------
bool bwd_mma_supported(Dims d) { return d.n == 4 && d.C % 8 == 0; }

int bwd_mma_kp(Dims d) { return (d.K() + 7) / 8 * 8; }
int bwd_mma_record_floats(Dims d) { return (d.n * d.n + 2 * d.n + 3 + 3) / 4 * 4; }

// token groups (of 16) per dx block: about one resident wave of 128-thread blocks
static int dx_groups_per_block(Dims d) {
    const int64_t colblocks = (d.C + kDxCols - 1) / kDxCols;
    const int64_t groups = (d.B + 15) / 16;
    int64_t want_blocks = 3 * 148;                       // three blocks per SM
    int64_t split = (want_blocks + colblocks - 1) / colblocks;
    if (split < 1) split = 1;
    int64_t gpb = (groups + split - 1) / split;
    gpb = (gpb + kDxWarps - 1) / kDxWarps * kDxWarps;     // every warp gets the same share
    if (gpb < kDxWarps) gpb = kDxWarps;
    return (int)gpb;
}

int dx_mma_token_blocks(Dims d) {
    const int64_t groups = (d.B + 15) / 16;
    const int gpb = dx_groups_per_block(d);
    return (int)((groups + gpb - 1) / gpb);
}

cudaError_t launch_dx_mma(bf16* dx, float* dw_part, const bf16* x, const bf16* g, const bf16* w,
                          const float* rec, const bf16* dprb, const bf16* phi, Dims d,
                          cudaStream_t s) {
    if (d.B == 0) return cudaSuccess;
    if (!bwd_mma_supported(d)) return cudaErrorNotSupported;
    const int gpb = dx_groups_per_block(d);
    const dim3 grid((unsigned)((d.C + kDxCols - 1) / kDxCols), (unsigned)dx_mma_token_blocks(d));
    const size_t smem = (size_t)2 * (4 * 4) * (kDxWarps * 32) * sizeof(uint4);   // 64 KB
    cudaError_t e = cudaFuncSetAttribute(dx_mma_kernel<4>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return e;
    dx_mma_kernel<4><<<grid, kDxWarps * 32, smem, s>>>(dx, dw_part, x, g, w, rec, dprb, phi, d.B,
                                                        d.C, gpb);
    return launched();
}

cudaError_t launch_dphi_mma(float* dphi, const bf16* x, const bf16* dprT, Dims d, cudaStream_t s) {
    const int K = d.K(), KP = bwd_mma_kp(d);
    const int64_t Bp = (d.B + 15) / 16 * 16;
    const int64_t nC = d.nC();
    constexpr int MT16 = 2;
    const dim3 grid((unsigned)((nC + kDphiCols - 1) / kDphiCols),
                    (unsigned)((KP + MT16 * 16 - 1) / (MT16 * 16)));
    dphi_mma_kernel<MT16><<<grid, kDphiWarps * 32, 0, s>>>(dphi, x, dprT, d.B, Bp, K, KP, nC);
    return launched();
}

}  // namespace mhc
