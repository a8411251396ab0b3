/* See naive_mhc.h.  Test infrastructure only. */
#include "naive_mhc.h"

#include <math.h>

static double sigmoid_(double t) { return 1.0 / (1.0 + exp(-t)); }

int naive_mhc_dynamic_forward(const double* x, const double* w, const double* phi,
                              const double* alpha, const double* bias, long B, int n, long C,
                              int iters, double eps, double* y) {
    if (n < 1 || n > 32) return -1;
    const long nC = (long)n * C;
    const int K = 2 * n + n * n;
    double p[2 * 32 + 32 * 32], hp[32], hq[32], M[32][32];
    for (long b = 0; b < B; ++b) {
        const double* xb = x + b * nC;
        double ss = 0.0;
        for (long m = 0; m < nC; ++m) ss += xb[m] * xb[m];
        const double r = sqrt(ss / (double)nC + eps);
        for (int k = 0; k < K; ++k) {
            const double* ph = phi + (long)k * nC;
            double s = 0.0;
            for (long m = 0; m < nC; ++m) s += xb[m] * ph[m];
            p[k] = s / r;
        }
        for (int i = 0; i < n; ++i) {
            hp[i] = sigmoid_(alpha[0] * p[i] + bias[i]);
            hq[i] = 2.0 * sigmoid_(alpha[1] * p[n + i] + bias[n + i]);
            for (int j = 0; j < n; ++j)
                M[i][j] = exp(alpha[2] * p[2 * n + i * n + j] + bias[2 * n + i * n + j]);
        }
        for (int t = 0; t < iters; ++t) {
            for (int i = 0; i < n; ++i) {
                double s = 0.0;
                for (int j = 0; j < n; ++j) s += M[i][j];
                for (int j = 0; j < n; ++j) M[i][j] /= (s + eps);
            }
            for (int j = 0; j < n; ++j) {
                double s = 0.0;
                for (int i = 0; i < n; ++i) s += M[i][j];
                for (int i = 0; i < n; ++i) M[i][j] /= (s + eps);
            }
        }
        double sa = 0.0;
        for (long c = 0; c < C; ++c) {
            double a = 0.0;
            for (int i = 0; i < n; ++i) a += hp[i] * xb[(long)i * C + c];
            sa += a * a;
        }
        const double rho = sqrt(sa / (double)C + eps);
        for (long c = 0; c < C; ++c) {
            double a = 0.0;
            for (int i = 0; i < n; ++i) a += hp[i] * xb[(long)i * C + c];
            const double yn = a / rho * w[c];
            for (int i = 0; i < n; ++i) {
                double s = hq[i] * yn;
                for (int j = 0; j < n; ++j) s += M[i][j] * xb[(long)j * C + c];
                y[b * nC + (long)i * C + c] = s;
            }
        }
    }
    return 0;
}
