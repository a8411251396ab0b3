// mhc_cuda: the C++ torch extension of this package.  Same function names as the reference's
// pybind module (src/python/bindings.cu:544-554 of AndreSlavescu/mHC.cu); each one checks its
// tensors, allocates outputs and the workspace with torch, takes the current CUDA stream and
// forwards to the C ABI of libmhc_b200.so (include/mhc_b200.h).  No kernels live here.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <vector>

#include "mhc_b200.h"

namespace {

using torch::Tensor;

void check(int st, const char* what) {
    TORCH_CHECK(st == MHC_OK, what, " failed: ", mhc_status_string(st),
                st == MHC_ERR_CUDA ? mhc_last_cuda_error() : "");
}

void need(const Tensor& t, const char* name) {
    TORCH_CHECK(t.is_cuda(), name, " must be a CUDA tensor (there is no CPU path)");
    TORCH_CHECK(t.is_contiguous(), name, " must be contiguous");
}

int dtype_tag(const Tensor& x) {
    if (x.scalar_type() == torch::kFloat32) return MHC_F32;
    if (x.scalar_type() == torch::kBFloat16) return MHC_BF16;
    TORCH_CHECK(false, "streams must be float32 or bfloat16");
    return -1;
}

mhc_stream_t stream() { return (mhc_stream_t)at::cuda::getCurrentCUDAStream().stream(); }

Tensor workspace(int op, int64_t B, int n, int64_t C, int iters, int tag, const Tensor& like) {
    const size_t bytes = mhc_workspace_bytes(op, B, n, C, iters, tag);
    TORCH_CHECK(bytes != (size_t)-1, "bad problem size");
    return torch::empty({(int64_t)bytes + 16}, like.options().dtype(torch::kUInt8));
}

// ---- stand-alone ops -----------------------------------------------------------------------
static bool is_rect(const Tensor& inp) {
    return inp.dim() == 2 && (inp.size(0) != inp.size(1) || inp.size(0) > 32);
}

Tensor sinkhorn_knopp_fwd(Tensor inp, int64_t iters, double eps) {
    need(inp, "inp");
    TORCH_CHECK(inp.scalar_type() == torch::kFloat32 && (inp.dim() == 2 || inp.dim() == 3),
                "sinkhorn expects fp32 [M,N] or [batch,n,n]");
    c10::cuda::CUDAGuard guard(inp.device());
    auto out = torch::empty_like(inp);
    if (is_rect(inp)) {   // one matrix the batched square kernels do not cover (M, N <= 128)
        check(mhc_sinkhorn_rect_fwd(out.data_ptr<float>(), inp.data_ptr<float>(), (int)inp.size(0),
                                    (int)inp.size(1), (int)iters, (float)eps, stream()),
              "mhc_sinkhorn_rect_fwd");
        return out;
    }
    TORCH_CHECK(inp.size(-1) == inp.size(-2), "batched sinkhorn expects square matrices");
    const int64_t batch = inp.dim() == 3 ? inp.size(0) : 1;
    check(mhc_sinkhorn_fwd(out.data_ptr<float>(), inp.data_ptr<float>(), batch, (int)inp.size(-1),
                           (int)iters, (float)eps, stream()),
          "mhc_sinkhorn_fwd");
    return out;
}

Tensor sinkhorn_knopp_bwd(Tensor grad, Tensor inp, int64_t iters, double eps) {
    need(grad, "grad");
    need(inp, "inp");
    c10::cuda::CUDAGuard guard(inp.device());
    if (is_rect(inp)) {
        auto d_rect = torch::empty_like(inp);
        auto wsr = workspace(MHC_OP_SINKHORN_RECT_BWD, inp.size(0), (int)inp.size(1), 0, (int)iters,
                             MHC_F32, inp);
        check(mhc_sinkhorn_rect_bwd(d_rect.data_ptr<float>(), grad.data_ptr<float>(),
                                    inp.data_ptr<float>(), (int)inp.size(0), (int)inp.size(1),
                                    (int)iters, (float)eps, wsr.data_ptr(), wsr.numel(), stream()),
              "mhc_sinkhorn_rect_bwd");
        return d_rect;
    }
    const int64_t batch = inp.dim() == 3 ? inp.size(0) : 1;
    const int n = (int)inp.size(-1);
    auto d_inp = torch::empty_like(inp);
    auto ws = workspace(MHC_OP_SINKHORN_BWD, batch, n, 0, (int)iters, MHC_F32, inp);
    check(mhc_sinkhorn_bwd(d_inp.data_ptr<float>(), grad.data_ptr<float>(), inp.data_ptr<float>(),
                           batch, n, (int)iters, (float)eps, ws.data_ptr(), ws.numel(), stream()),
          "mhc_sinkhorn_bwd");
    return d_inp;
}

std::vector<Tensor> rmsnorm_fwd(Tensor inp, Tensor weight, double eps) {
    need(inp, "inp");
    need(weight, "weight");
    TORCH_CHECK(inp.scalar_type() == torch::kBFloat16 && weight.scalar_type() == torch::kBFloat16,
                "rmsnorm works on bf16");
    c10::cuda::CUDAGuard guard(inp.device());
    const int64_t B = inp.size(0), C = inp.size(1);
    auto out = torch::empty_like(inp);
    auto rms = torch::empty({B}, inp.options().dtype(torch::kFloat32));
    check(mhc_rmsnorm_fwd(out.data_ptr(), rms.data_ptr<float>(), inp.data_ptr(), weight.data_ptr(),
                          B, C, (float)eps, stream()),
          "mhc_rmsnorm_fwd");
    return {out, rms};
}

std::vector<Tensor> rmsnorm_bwd(Tensor grad, Tensor inp, Tensor weight, Tensor rms) {
    need(grad, "grad");
    need(inp, "inp");
    need(weight, "weight");
    need(rms, "rms");
    c10::cuda::CUDAGuard guard(inp.device());
    const int64_t B = inp.size(0), C = inp.size(1);
    auto d_inp = torch::empty_like(inp);
    auto d_w = torch::empty({C}, inp.options().dtype(torch::kFloat32));
    auto ws = workspace(MHC_OP_RMSNORM_BWD, B, 1, C, 0, MHC_BF16, inp);
    check(mhc_rmsnorm_bwd(d_inp.data_ptr(), d_w.data_ptr<float>(), grad.data_ptr(), inp.data_ptr(),
                          weight.data_ptr(), rms.data_ptr<float>(), B, C, ws.data_ptr(), ws.numel(),
                          stream()),
          "mhc_rmsnorm_bwd");
    return {d_inp, d_w};
}

// ---- static-H layer --------------------------------------------------------------------------
// returns (y, rms, H_pre_act, H_post_act, M)
std::vector<Tensor> mhc_layer_fwd(Tensor x, Tensor w, Tensor H_pre, Tensor H_post, Tensor H_res,
                                  int64_t iters, double eps) {
    need(x, "x_expanded"); need(w, "rmsnorm_weight"); need(H_pre, "H_pre"); need(H_post, "H_post");
    need(H_res, "H_res");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.size(0), n = x.size(1), C = x.size(2);
    const int tag = dtype_tag(x);
    auto f32 = x.options().dtype(torch::kFloat32);
    auto y = torch::empty_like(x);
    auto rms = torch::empty({B}, f32);
    auto hp = torch::empty({n}, f32), hq = torch::empty({n}, f32), M = torch::empty({n, n}, f32);
    auto ws = workspace(MHC_OP_STATIC_FWD, B, (int)n, C, (int)iters, tag, x);
    check(mhc_static_fwd(y.data_ptr(), rms.data_ptr<float>(), hp.data_ptr<float>(),
                         hq.data_ptr<float>(), M.data_ptr<float>(), x.data_ptr(), w.data_ptr(),
                         H_pre.data_ptr<float>(), H_post.data_ptr<float>(), H_res.data_ptr<float>(),
                         B, (int)n, C, (int)iters, (float)eps, tag, ws.data_ptr(), ws.numel(),
                         stream()),
          "mhc_static_fwd");
    return {y, rms, hp, hq, M};
}

Tensor mhc_layer_fwd_inference(Tensor x, Tensor w, Tensor H_pre, Tensor H_post, Tensor H_res,
                               int64_t iters, double eps) {
    need(x, "x_expanded"); need(w, "rmsnorm_weight");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.size(0), n = x.size(1), C = x.size(2);
    const int tag = dtype_tag(x);
    auto y = torch::empty_like(x);
    auto ws = workspace(MHC_OP_STATIC_FWD, B, (int)n, C, (int)iters, tag, x);
    check(mhc_static_fwd(y.data_ptr(), nullptr, nullptr, nullptr, nullptr, x.data_ptr(),
                         w.data_ptr(), H_pre.data_ptr<float>(), H_post.data_ptr<float>(),
                         H_res.data_ptr<float>(), B, (int)n, C, (int)iters, (float)eps, tag,
                         ws.data_ptr(), ws.numel(), stream()),
          "mhc_static_fwd (inference)");
    return y;
}

// returns (dx, d_rmsnorm_weight, d_H_pre, d_H_post, d_H_res)
std::vector<Tensor> mhc_layer_bwd(Tensor dy, Tensor x, Tensor w, Tensor H_res, Tensor rms, Tensor hp,
                                  Tensor hq, Tensor M, int64_t iters, double eps) {
    need(dy, "grad_output"); need(x, "x_expanded");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.size(0), n = x.size(1), C = x.size(2);
    const int tag = dtype_tag(x);
    auto f32 = x.options().dtype(torch::kFloat32);
    auto dx = torch::empty_like(x);
    auto d_w = torch::empty({C}, f32), d_hp = torch::empty({n}, f32), d_hq = torch::empty({n}, f32),
         d_hr = torch::empty({n, n}, f32);
    auto ws = workspace(MHC_OP_STATIC_BWD, B, (int)n, C, (int)iters, tag, x);
    check(mhc_static_bwd(dx.data_ptr(), d_w.data_ptr<float>(), d_hp.data_ptr<float>(),
                         d_hq.data_ptr<float>(), d_hr.data_ptr<float>(), dy.data_ptr(), x.data_ptr(),
                         w.data_ptr(), H_res.data_ptr<float>(), rms.data_ptr<float>(),
                         hp.data_ptr<float>(), hq.data_ptr<float>(), M.data_ptr<float>(), B, (int)n, C,
                         (int)iters, (float)eps, tag, ws.data_ptr(), ws.numel(), stream()),
          "mhc_static_bwd");
    return {dx, d_w, d_hp, d_hq, d_hr};
}

// ---- dynamic-H layer -------------------------------------------------------------------------
// phi [K, nC] in x's dtype (rows pre, post, res); alpha [3], bias [K] fp32 on the device.
// returns (y, rms, rms_h, H_pre, H_post, M, proj, sk_den)
std::vector<Tensor> mhc_layer_fwd_dynamic(Tensor x, Tensor w, Tensor phi, Tensor alpha, Tensor bias,
                                          int64_t iters, double eps) {
    need(x, "x_expanded"); need(w, "rmsnorm_weight"); need(phi, "phi"); need(alpha, "alpha");
    need(bias, "bias");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.size(0), n = x.size(1), C = x.size(2), K = 2 * n + n * n;
    const int tag = dtype_tag(x);
    TORCH_CHECK(phi.scalar_type() == x.scalar_type() && phi.numel() == K * n * C,
                "phi must be [K, nC] in the dtype of x");
    auto f32 = x.options().dtype(torch::kFloat32);
    auto y = torch::empty_like(x);
    auto rms = torch::empty({B}, f32), rms_h = torch::empty({B}, f32);
    auto hp = torch::empty({B, n}, f32), hq = torch::empty({B, n}, f32);
    auto M = torch::empty({B, n, n}, f32), proj = torch::empty({B, K}, f32);
    auto den = torch::empty({B, 2 * iters, n <= 4 ? 4 : 8}, f32);
    auto ws = workspace(MHC_OP_DYNAMIC_FWD, B, (int)n, C, (int)iters, tag, x);
    check(mhc_dynamic_fwd(y.data_ptr(), rms.data_ptr<float>(), rms_h.data_ptr<float>(),
                          hp.data_ptr<float>(), hq.data_ptr<float>(), M.data_ptr<float>(),
                          proj.data_ptr<float>(), den.data_ptr<float>(), x.data_ptr(), w.data_ptr(),
                          phi.data_ptr(), alpha.data_ptr<float>(), bias.data_ptr<float>(), B, (int)n,
                          C, (int)iters, (float)eps, tag, ws.data_ptr(), ws.numel(), stream()),
          "mhc_dynamic_fwd");
    return {y, rms, rms_h, hp, hq, M, proj, den};
}

// returns (dx, d_rmsnorm_weight [C], d_phi [K,nC], d_alpha [3], d_bias [K]), gradients fp32
std::vector<Tensor> mhc_layer_bwd_dynamic(Tensor dy, Tensor x, Tensor w, Tensor phi, Tensor alpha,
                                          Tensor bias, Tensor rms, Tensor rms_h, Tensor hp, Tensor hq,
                                          Tensor M, Tensor proj, Tensor den, int64_t iters,
                                          double eps) {
    need(dy, "grad_output"); need(x, "x_expanded");
    c10::cuda::CUDAGuard guard(x.device());
    const int64_t B = x.size(0), n = x.size(1), C = x.size(2), K = 2 * n + n * n;
    const int tag = dtype_tag(x);
    auto f32 = x.options().dtype(torch::kFloat32);
    auto dx = torch::empty_like(x);
    auto d_w = torch::empty({C}, f32), d_phi = torch::empty({K, n * C}, f32),
         d_alpha = torch::empty({3}, f32), d_bias = torch::empty({K}, f32);
    auto ws = workspace(MHC_OP_DYNAMIC_BWD, B, (int)n, C, (int)iters, tag, x);
    check(mhc_dynamic_bwd(dx.data_ptr(), d_w.data_ptr<float>(), d_phi.data_ptr<float>(),
                          d_alpha.data_ptr<float>(), d_bias.data_ptr<float>(), dy.data_ptr(),
                          x.data_ptr(), w.data_ptr(), phi.data_ptr(), alpha.data_ptr<float>(),
                          bias.data_ptr<float>(), rms.data_ptr<float>(), rms_h.data_ptr<float>(),
                          hp.data_ptr<float>(), hq.data_ptr<float>(), M.data_ptr<float>(),
                          proj.data_ptr<float>(), den.data_ptr<float>(), B, (int)n, C, (int)iters,
                          (float)eps, tag, ws.data_ptr(), ws.numel(), stream()),
          "mhc_dynamic_bwd");
    return {dx, d_w, d_phi, d_alpha, d_bias};
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.doc() = "mHC layer for B200: torch front end of libmhc_b200.so";
    m.def("sinkhorn_knopp_fwd", &sinkhorn_knopp_fwd);
    m.def("sinkhorn_knopp_bwd", &sinkhorn_knopp_bwd);
    m.def("rmsnorm_fwd", &rmsnorm_fwd);
    m.def("rmsnorm_bwd", &rmsnorm_bwd);
    m.def("mhc_layer_fwd", &mhc_layer_fwd);
    m.def("mhc_layer_fwd_inference", &mhc_layer_fwd_inference);
    m.def("mhc_layer_bwd", &mhc_layer_bwd);
    m.def("mhc_layer_fwd_dynamic", &mhc_layer_fwd_dynamic);
    m.def("mhc_layer_bwd_dynamic", &mhc_layer_bwd_dynamic);
    m.def("abi_version", []() { return mhc_abi_version(); });
    m.def("kernels_enqueued", []() { return (uint64_t)mhc_kernels_enqueued(); });
}
