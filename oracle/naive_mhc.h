/* CPU restatement in plain C of the reference's naive dynamic-H mHC layer forward — TEST
 * INFRASTRUCTURE ONLY (the checker of the native, torch-free tests; never linked into the product
 * library).  Follows _naive_mhc_dynamic / NaiveMHCLayerDynamic of AndreSlavescu/mHC.cu
 * (src/python/tests/test_layer.py:7-50, src/python/benchmarks/bench_layer.py:90-145):
 *
 *   r = sqrt(mean(x_flat^2) + eps)          p = (x_flat / r) phi^T              [B, K], K = 2n + n^2
 *   H_pre = sigmoid(a0 p_pre + b_pre)       H_post = 2 sigmoid(a1 p_post + b_post)
 *   M = Sinkhorn(exp(a2 p_res + b_res)):    iters x { M /= rowsum + eps ; M /= colsum + eps }
 *   a = sum_i H_pre[i] x[i,:]   rho = sqrt(mean(a^2) + eps)   y[i,:] = sum_j M[i,j] x[j,:] + H_post[i] a / rho * w
 *
 * Pinned against the golden vectors drawn from the reference's own code: tests/test_oracle_golden.py
 * calls this function through ctypes and compares it with tests/golden/dyn*.npz.
 *
 * x [B][n][C], w [C], phi [K][n*C] (rows pre[n], post[n], res[n*n]), alpha [3], bias [K]; y [B][n][C].
 * Everything double.  Returns 0, or -1 if n > 32. */
#ifndef ORACLE_NAIVE_MHC_H
#define ORACLE_NAIVE_MHC_H

#ifdef __cplusplus
extern "C" {
#endif

int naive_mhc_dynamic_forward(const double* x, const double* w, const double* phi,
                              const double* alpha, const double* bias, long B, int n, long C,
                              int iters, double eps, double* y);

#ifdef __cplusplus
}
#endif
#endif
