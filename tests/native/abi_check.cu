// Torch-free check and timing of the C ABI (include/mhc_b200.h): plain CUDA runtime, raw device
// buffers, the same calls a native consumer of the library makes.  Mirrors what the reference's
// own native harnesses do over its kernels (src/csrc/tests/test_mhc_layer.cu,
// src/csrc/benchmarks/bench_mhc_layer.cu), but against the CPU restatement in oracle/naive_mhc.c.
//
//   abi_check            fp32 streams, B=6 n=4 C=40: y against the C oracle (1e-5), then d_bias,
//                        d_alpha and samples of d_phi, dx against central differences of the oracle
//                        loss  L = sum(y * dy)  (5e-4: the differences are taken in fp64 on the
//                        oracle, the analytic gradients come from the fp32 kernels)
//   abi_check --bench    bf16 streams, B=1280 n=4 C=2560: forward + backward captured into a CUDA
//                        graph, 200 replays over four input sets, microseconds per step
//
// Exit code 0 = all checks passed.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/mhc_b200.h"
#include "../../oracle/naive_mhc.h"

#define CK(call)                                                                          \
    do {                                                                                  \
        cudaError_t e_ = (call);                                                          \
        if (e_ != cudaSuccess) {                                                          \
            std::fprintf(stderr, "%s:%d: %s\n", __FILE__, __LINE__, cudaGetErrorString(e_)); \
            std::exit(2);                                                                 \
        }                                                                                 \
    } while (0)
#define MHC(call)                                                                         \
    do {                                                                                  \
        int s_ = (call);                                                                  \
        if (s_ != MHC_OK) {                                                               \
            std::fprintf(stderr, "%s:%d: %s (%s)\n", __FILE__, __LINE__, mhc_status_string(s_), \
                         mhc_last_cuda_error());                                          \
            std::exit(2);                                                                 \
        }                                                                                 \
    } while (0)

namespace {

// deterministic pseudo-normal numbers (sum of uniforms), no library dependence
struct Rng {
    uint64_t s;
    explicit Rng(uint64_t seed) : s(seed * 0x9E3779B97F4A7C15ull + 1) {}
    double uni() {
        s = s * 6364136223846793005ull + 1442695040888963407ull;
        return (double)(s >> 11) / 9007199254740992.0;
    }
    double normal() {
        double t = 0.0;
        for (int i = 0; i < 12; ++i) t += uni();
        return t - 6.0;
    }
};

template <typename T>
T* dev_alloc(size_t count) {
    void* p = nullptr;
    CK(cudaMalloc(&p, (count ? count : 1) * sizeof(T)));
    return static_cast<T*>(p);
}

struct Problem {
    long B, C;
    int n, K, iters;
    double eps;
    std::vector<double> x, dy, w, phi, alpha, bias;
    Problem(long B_, int n_, long C_, int iters_, double eps_, uint64_t seed)
        : B(B_), C(C_), n(n_), K(2 * n_ + n_ * n_), iters(iters_), eps(eps_) {
        Rng r(seed);
        x.resize(B * n * C);
        dy.resize(B * n * C);
        w.resize(C);
        phi.resize((size_t)K * n * C);
        alpha = {0.5, 0.4, 0.3};
        bias.resize(K);
        for (auto& v : x) v = (double)(float)r.normal();
        for (auto& v : dy) v = (double)(float)r.normal();
        // the weight is a bf16 parameter of the layer: keep it exactly representable
        for (auto& v : w) v = (double)__bfloat162float(__float2bfloat16((float)(1.0 + 0.25 * r.normal())));
        for (auto& v : phi) v = (double)(float)(0.05 * r.normal());
        for (auto& v : bias) v = (double)(float)(0.3 * r.normal());
    }
    double loss() const {   // L = sum(y * dy) on the oracle
        std::vector<double> y(x.size());
        naive_mhc_dynamic_forward(x.data(), w.data(), phi.data(), alpha.data(), bias.data(), B, n, C,
                                  iters, eps, y.data());
        double L = 0.0;
        for (size_t i = 0; i < y.size(); ++i) L += y[i] * dy[i];
        return L;
    }
};

template <typename T>
std::vector<T> to_float_like(const std::vector<double>& v);
template <>
std::vector<float> to_float_like<float>(const std::vector<double>& v) {
    return std::vector<float>(v.begin(), v.end());
}
template <>
std::vector<__nv_bfloat16> to_float_like<__nv_bfloat16>(const std::vector<double>& v) {
    std::vector<__nv_bfloat16> o(v.size());
    for (size_t i = 0; i < v.size(); ++i) o[i] = __float2bfloat16((float)v[i]);
    return o;
}

template <typename T>
T* upload(const std::vector<T>& h) {
    T* d = dev_alloc<T>(h.size());
    CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice));
    return d;
}

struct DeviceLayer {   // everything one dynamic forward + backward needs, on the device
    long B, C;
    int n, K, iters, dtype;
    float eps;
    void *x, *dy, *y, *dx, *phi, *w;
    float *alpha, *bias, *rms, *rms_h, *H_pre, *H_post, *M, *proj, *sk_den;
    float *d_w, *d_phi, *d_alpha, *d_bias;
    void *ws_f, *ws_b;
    size_t ws_f_bytes, ws_b_bytes;
};

template <typename T>
DeviceLayer make_device(const Problem& p, int dtype) {
    DeviceLayer d{};
    d.B = p.B; d.C = p.C; d.n = p.n; d.K = p.K; d.iters = p.iters; d.dtype = dtype; d.eps = (float)p.eps;
    const size_t ne = (size_t)p.B * p.n * p.C;
    d.x = upload(to_float_like<T>(p.x));
    d.dy = upload(to_float_like<T>(p.dy));
    d.phi = upload(to_float_like<T>(p.phi));
    d.w = upload(to_float_like<__nv_bfloat16>(p.w));
    d.y = dev_alloc<T>(ne);
    d.dx = dev_alloc<T>(ne);
    d.alpha = upload(to_float_like<float>(p.alpha));
    d.bias = upload(to_float_like<float>(p.bias));
    d.rms = dev_alloc<float>(p.B); d.rms_h = dev_alloc<float>(p.B);
    d.H_pre = dev_alloc<float>(p.B * p.n); d.H_post = dev_alloc<float>(p.B * p.n);
    d.M = dev_alloc<float>(p.B * p.n * p.n); d.proj = dev_alloc<float>(p.B * p.K);
    d.sk_den = dev_alloc<float>((size_t)p.B * 2 * p.iters * (p.n <= 4 ? 4 : 8));
    d.d_w = dev_alloc<float>(p.C); d.d_phi = dev_alloc<float>((size_t)p.K * p.n * p.C);
    d.d_alpha = dev_alloc<float>(3); d.d_bias = dev_alloc<float>(p.K);
    d.ws_f_bytes = mhc_workspace_bytes(MHC_OP_DYNAMIC_FWD, p.B, p.n, p.C, p.iters, dtype);
    d.ws_b_bytes = mhc_workspace_bytes(MHC_OP_DYNAMIC_BWD, p.B, p.n, p.C, p.iters, dtype);
    d.ws_f = dev_alloc<char>(d.ws_f_bytes + 256);
    d.ws_b = dev_alloc<char>(d.ws_b_bytes + 256);
    return d;
}

void run_step(const DeviceLayer& d, const void* x, const void* dy, cudaStream_t s) {
    MHC(mhc_dynamic_fwd(d.y, d.rms, d.rms_h, d.H_pre, d.H_post, d.M, d.proj, d.sk_den, x, d.w, d.phi,
                        d.alpha, d.bias, d.B, d.n, d.C, d.iters, d.eps, d.dtype, d.ws_f,
                        d.ws_f_bytes + 256, s));
    MHC(mhc_dynamic_bwd(d.dx, d.d_w, d.d_phi, d.d_alpha, d.d_bias, dy, x, d.w, d.phi, d.alpha, d.bias,
                        d.rms, d.rms_h, d.H_pre, d.H_post, d.M, d.proj, d.sk_den, d.B, d.n, d.C,
                        d.iters, d.eps, d.dtype, d.ws_b, d.ws_b_bytes + 256, s));
}

int check() {
    Problem p(6, 4, 40, 20, 1e-5, 7);
    DeviceLayer d = make_device<float>(p, MHC_F32);
    run_step(d, d.x, d.dy, nullptr);
    CK(cudaDeviceSynchronize());
    const size_t ne = p.x.size();
    std::vector<float> y(ne), dx(ne), dphi((size_t)p.K * p.n * p.C), dbias(p.K), dalpha(3);
    CK(cudaMemcpy(y.data(), d.y, ne * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dx.data(), d.dx, ne * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dphi.data(), d.d_phi, dphi.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dbias.data(), d.d_bias, dbias.size() * 4, cudaMemcpyDeviceToHost));
    CK(cudaMemcpy(dalpha.data(), d.d_alpha, 12, cudaMemcpyDeviceToHost));

    int bad = 0;
    {   // forward
        std::vector<double> ref(ne);
        naive_mhc_dynamic_forward(p.x.data(), p.w.data(), p.phi.data(), p.alpha.data(), p.bias.data(),
                                  p.B, p.n, p.C, p.iters, p.eps, ref.data());
        double num = 0.0, den = 0.0;
        for (size_t i = 0; i < ne; ++i) {
            num = std::fmax(num, std::fabs((double)y[i] - ref[i]));
            den = std::fmax(den, std::fabs(ref[i]));
        }
        std::printf("forward y: max|a-b|/max|b| = %.3g (bar 1e-5)\n", num / den);
        if (!(num / den <= 1e-5)) ++bad;
    }
    // gradients against central differences of the oracle loss
    enum Which { kBias, kAlpha, kPhi, kX };
    auto fd = [&](Which which, size_t idx, double h) {
        Problem q = p;
        std::vector<double>& a = which == kBias ? q.bias : which == kAlpha ? q.alpha
                               : which == kPhi ? q.phi : q.x;
        const double v0 = a[idx];
        a[idx] = v0 + h;
        const double lp = q.loss();
        a[idx] = v0 - h;
        const double lm = q.loss();
        return (lp - lm) / (2 * h);
    };
    auto report = [&](const char* what, double got, double want, double scale) {
        const double err = std::fabs(got - want) / scale;
        std::printf("%-10s analytic % .6e  finite-diff % .6e  err/scale %.2g\n", what, got, want, err);
        if (!(err <= 5e-4)) ++bad;
    };
    double sb = 0.0;
    for (float v : dbias) sb = std::fmax(sb, std::fabs((double)v));
    for (int k : {0, 5, 9, 23}) report("d_bias", dbias[k], fd(kBias, k, 1e-5), sb);
    double sa = std::fmax(std::fabs((double)dalpha[0]), std::fmax(std::fabs((double)dalpha[1]),
                                                                 std::fabs((double)dalpha[2])));
    for (int k = 0; k < 3; ++k) report("d_alpha", dalpha[k], fd(kAlpha, k, 1e-5), sa);
    double sp = 0.0, sx = 0.0;
    for (float v : dphi) sp = std::fmax(sp, std::fabs((double)v));
    for (float v : dx) sx = std::fmax(sx, std::fabs((double)v));
    for (size_t idx : {size_t(3), size_t(5 * 160 + 77), size_t(20 * 160 + 159)})
        report("d_phi", dphi[idx], fd(kPhi, idx, 1e-5), sp);
    for (size_t idx : {size_t(0), size_t(2 * 160 + 41), ne - 1}) report("dx", dx[idx], fd(kX, idx, 1e-5), sx);
    std::printf("kernels enqueued by the library: %llu\n", mhc_kernels_enqueued());
    std::printf(bad ? "FAILED (%d checks)\n" : "PASSED\n", bad);
    return bad ? 1 : 0;
}

int bench() {
    const int R = 4, steps = 200;
    Problem p(1280, 4, 2560, 20, 1e-6, 1);
    for (auto& v : p.alpha) v = 0.01;
    for (auto& v : p.bias) v = 0.0;
    DeviceLayer d = make_device<__nv_bfloat16>(p, MHC_BF16);
    // four input sets (420 MB of streams together with their outputs) so that steps do not reuse L2
    const size_t ne = p.x.size();
    std::vector<void*> xs(R), dys(R);
    for (int r = 0; r < R; ++r) {
        xs[r] = dev_alloc<__nv_bfloat16>(ne);
        dys[r] = dev_alloc<__nv_bfloat16>(ne);
        CK(cudaMemcpy(xs[r], d.x, ne * 2, cudaMemcpyDeviceToDevice));
        CK(cudaMemcpy(dys[r], d.dy, ne * 2, cudaMemcpyDeviceToDevice));
    }
    cudaStream_t s;
    CK(cudaStreamCreate(&s));
    for (int r = 0; r < R; ++r) run_step(d, xs[r], dys[r], s);   // warm-up, attribute set-up
    CK(cudaStreamSynchronize(s));
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    CK(cudaStreamBeginCapture(s, cudaStreamCaptureModeThreadLocal));
    for (int r = 0; r < R; ++r) run_step(d, xs[r], dys[r], s);
    CK(cudaStreamEndCapture(s, &graph));
    CK(cudaGraphInstantiate(&exec, graph, 0));
    for (int i = 0; i < 5; ++i) CK(cudaGraphLaunch(exec, s));
    CK(cudaStreamSynchronize(s));
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0));
    CK(cudaEventCreate(&e1));
    CK(cudaEventRecord(e0, s));
    for (int i = 0; i < steps / R; ++i) CK(cudaGraphLaunch(exec, s));
    CK(cudaEventRecord(e1, s));
    CK(cudaEventSynchronize(e1));
    float ms = 0.f;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    const double us = ms * 1e3 / steps;
    std::printf("c3 (B=1280 n=4 C=2560 bf16) forward+backward through the C ABI, CUDA graph replay: "
                "%.1f us per step, %.2f M tokens/s\n", us, 1280.0 / us);
    return 0;
}

}  // namespace

int main(int argc, char** argv) {
    if (mhc_abi_version() < 2) {
        std::fprintf(stderr, "library ABI too old\n");
        return 2;
    }
    if (argc > 1 && std::strcmp(argv[1], "--bench") == 0) return bench();
    return check();
}
