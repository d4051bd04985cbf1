/*
 * Plain-C restatement of the attention column mean.  TEST INFRASTRUCTURE ONLY:
 * it is loaded by the tests, the smoke test and the CPU-baseline leg of the
 * benchmark, never by the product path.
 *
 * Definition followed (reference flash_colsum/baselines.py:35-78):
 *   s[q][k]  = scale * <Q[b,h,q,:], K[b,h,k,:]>                 (:42)
 *   causal:    s[q][k] = -inf unless k <= max(0, Sk - Sq) + q    (:49-63)
 *   p[q][:]  = softmax over k of s[q][:]                         (:66)
 *   out[b,k] = mean over h and over the first `rows` query rows  (:68-76)
 * where rows = Sq, or min(cls_len, Sq) for the non-causal CLS-prefix case.
 *
 * Inputs are fp32 (callers upcast fp16/bf16 first so that both sides of a parity
 * check see the same values); all arithmetic here is double.  Parallel over
 * (b, h) when built with -fopenmp.
 */
#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int colsum_oracle_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Returns 0, or -1 on bad arguments / allocation failure. `out` is (B, Sk) doubles. */
int colsum_oracle_f32(const float *q, const float *k, double *out,
                      int B, int H, int Sq, int Sk, int D,
                      double scale, int is_causal, int cls_len) {
    if (!q || !k || !out || B <= 0 || H <= 0 || Sq <= 0 || Sk <= 0 || D <= 0) return -1;
    int rows = Sq;
    if (!is_causal && cls_len > 0 && cls_len < Sq) rows = cls_len;
    const int k_past = Sk > Sq ? Sk - Sq : 0;
    const long n_out = (long)B * Sk;
    memset(out, 0, sizeof(double) * (size_t)n_out);
    int failed = 0;

#pragma omp parallel
    {
        double *local = (double *)calloc((size_t)n_out, sizeof(double));
        double *s = (double *)malloc(sizeof(double) * (size_t)Sk);
        if (!local || !s) {
#pragma omp atomic write
            failed = 1;
        } else {
#pragma omp for schedule(dynamic, 1) collapse(2)
            for (int b = 0; b < B; ++b) {
                for (int h = 0; h < H; ++h) {
                    const float *qh = q + ((size_t)b * H + h) * (size_t)Sq * D;
                    const float *kh = k + ((size_t)b * H + h) * (size_t)Sk * D;
                    double *o = local + (size_t)b * Sk;
                    for (int r = 0; r < rows; ++r) {
                        const float *qr = qh + (size_t)r * D;
                        int last = is_causal ? k_past + r : Sk - 1;
                        if (last > Sk - 1) last = Sk - 1;
                        double m = -INFINITY;
                        for (int j = 0; j <= last; ++j) {
                            const float *kr = kh + (size_t)j * D;
                            double acc = 0.0;
                            for (int d = 0; d < D; ++d) acc += (double)qr[d] * (double)kr[d];
                            acc *= scale;
                            s[j] = acc;
                            if (acc > m) m = acc;
                        }
                        double l = 0.0;
                        for (int j = 0; j <= last; ++j) {
                            s[j] = exp(s[j] - m);
                            l += s[j];
                        }
                        const double inv = 1.0 / l;
                        for (int j = 0; j <= last; ++j) o[j] += s[j] * inv;
                    }
                }
            }
#pragma omp critical
            {
                for (long i = 0; i < n_out; ++i) out[i] += local[i];
            }
        }
        free(local);
        free(s);
    }
    if (failed) return -1;
    const double norm = 1.0 / ((double)H * (double)rows);
    for (long i = 0; i < n_out; ++i) out[i] *= norm;
    return 0;
}
