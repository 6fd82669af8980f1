/*
 * Scalar C restatement of the kermac fused-distance operators.  TEST INFRASTRUCTURE
 * ONLY: an independent second statement of oracle/kermac_oracle.py, written as the
 * plain loops the reference documents, in double precision from float inputs.
 *
 *   km_oracle_build : README.md:80-92 (c-style cdist loop) generalised with the
 *                     operator chain of include/build_a_kernel.cuh:339-447
 *   km_oracle_grad  : README.md:122-134 (c-style gradient loop); the sign is
 *                     copysign(1, float difference) as in
 *                     include/kermac_internal_common.cuh:178-192
 *
 * Enum values: inner_op 0 = DIFF, 1 = DOT; power 0 = NOOP, 1 = ABS, 2 = SQUARE,
 * 3 = SQRT, 4 = POW; kernel 0 = NONE, 1 = LAPLACE, 2 = GAUSSIAN.
 * Parity pin: see the header of oracle/kermac_oracle.py.
 */
#include <math.h>
#include <stddef.h>

static double apply_power(double x, int kind, double p, int inner) {
    switch (kind) {
        case 1: return fabs(x);
        case 2: return x * x;
        case 3: return sqrt(x);
        case 4: return pow(inner ? fabs(x) : x, p);
        default: return x;
    }
}

/* out[m * N + n] (row-major M x N doubles); a[m * a_sm + k * a_sk], b[n * b_sn + k * b_sk] */
void km_oracle_build(const float* a, const float* b, double* out, int M, int N, int K, long a_sm, long a_sk,
                     long b_sn, long b_sk, int inner_op, int inner_power, int outer_power, int kernel_type,
                     double p_inner, double p_outer, double bandwidth, double epsilon, double regularization,
                     int reg_off_x, int reg_off_y) {
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            double acc = 0.0;
            for (int k = 0; k < K; k++) {
                double av = (double)a[m * a_sm + k * a_sk];
                double bv = (double)b[n * b_sn + k * b_sk];
                double x  = inner_op == 0 ? bv - av : bv * av;
                acc += apply_power(x, inner_power, p_inner, 1);
            }
            acc = apply_power(acc, outer_power, p_outer, 0);
            if (kernel_type != 0) {
                if (acc < epsilon) acc = 0.0;
                double gamma = kernel_type == 1 ? 1.0 / bandwidth : 1.0 / (2.0 * bandwidth * bandwidth);
                acc = exp(-acc * gamma);
                if (regularization != 0.0 && reg_off_x + m == reg_off_y + n) acc = 1.0 + regularization;
            }
            out[(size_t)m * N + n] = acc;
        }
    }
}

/* a[k * lda + m], b[n * ldb + k], c[o * ldc + k], d[n * ldd + m], out[(o * N + n) * M + m] */
void km_oracle_grad(const float* a, const float* b, const float* c, const float* d, double* out, int M, int N, int O,
                    int K, long lda, long ldb, long ldc, long ldd, double p) {
    for (int m = 0; m < M; m++) {
        for (int n = 0; n < N; n++) {
            for (int o = 0; o < O; o++) {
                double acc = 0.0;
                for (int k = 0; k < K; k++) {
                    float  diff_f = d[n * ldd + m] - b[n * ldb + k];
                    double sign   = (double)copysignf(1.0f, diff_f);
                    double mag    = fabs((double)d[n * ldd + m] - (double)b[n * ldb + k]);
                    double g      = p == 1.0 ? sign : (p == 2.0 ? sign * mag : sign * pow(mag, p - 1.0));
                    acc += (double)c[o * ldc + k] * (double)a[k * lda + m] * g;
                }
                out[((size_t)o * N + n) * M + m] = acc;
            }
        }
    }
}
