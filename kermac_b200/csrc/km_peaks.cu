// Register-only microbenchmarks of the arithmetic pipes the distance kernels are
// bound by.  They give the roofline denominators (fp32 lane-operations per second,
// MUFU operations per second) for the device and clock the benchmark actually
// runs at, instead of a nominal figure.
#include "km_common.cuh"
#include "km_host.h"

namespace km {
namespace {

constexpr int PEAK_THREADS = 256;
constexpr int PEAK_CHAINS  = 16;   // independent dependency chains per thread

// kind 0: scalar fma chain, kind 1: packed fma chain, kind 2: lg2+ex2 chain,
// kind 3: sub + add|.| chain (two dependent scalar adds per step).
template <int KIND>
__global__ void __launch_bounds__(PEAK_THREADS) pipe_kernel(float* sink, int iterations, float seed) {
    float x[PEAK_CHAINS];
    u64   y[PEAK_CHAINS];
#pragma unroll
    for (int i = 0; i < PEAK_CHAINS; ++i) {
        x[i] = seed + 0.001f * (threadIdx.x + i);
        y[i] = pack2(x[i], x[i] + 0.5f);
    }
    const float mulc = 0.999f, addc = 0.001f;
    const u64   mul2c = pack2(mulc, mulc), add2c = pack2(addc, addc);
    for (int it = 0; it < iterations; ++it) {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
#pragma unroll
            for (int i = 0; i < PEAK_CHAINS; ++i) {
                if constexpr (KIND == 0) {
                    x[i] = fmaf(x[i], mulc, addc);
                } else if constexpr (KIND == 1) {
                    y[i] = fma2(y[i], mul2c, add2c);
                } else if constexpr (KIND == 2) {
                    x[i] = ex2_approx(lg2_approx(x[i]));
                } else {
                    const float d = x[(i + 1) % PEAK_CHAINS] - seed;
                    x[i] += fabsf(d);
                }
            }
        }
    }
    float s = 0.0f;
#pragma unroll
    for (int i = 0; i < PEAK_CHAINS; ++i) {
        float lo, hi;
        unpack2(y[i], lo, hi);
        s += x[i] + lo + hi;
    }
    if (s == 123.456f) sink[0] = s;   // keeps the chains alive without a store in practice
}

typedef void (*PipeFn)(float*, int, float);

}  // namespace
}  // namespace km

extern "C" int kermac_b200_measure_pipe(int32_t kind, int32_t iterations, double* ops_per_second,
                                        double* milliseconds) {
    using namespace km;
    if (!ops_per_second) return fail(KM_ERR_NULL_POINTER, "ops_per_second is NULL");
    if (kind < 0 || kind > 3) return fail(KM_ERR_BAD_ENUM, "kind %d is not a pipe benchmark", kind);
    if (iterations < 1 || iterations > (1 << 24)) return fail(KM_ERR_BAD_SHAPE, "iterations out of range");
    if (int rc = require_sm100()) return rc;
    PipeFn fns[4] = {pipe_kernel<0>, pipe_kernel<1>, pipe_kernel<2>, pipe_kernel<3>};
    float* sink   = nullptr;
    if (int rc = cuda_status(cudaMalloc(&sink, 256), "cudaMalloc")) return rc;
    const int blocks = sm_count() * 8;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    fns[kind]<<<blocks, PEAK_THREADS>>>(sink, iterations / 8 + 1, 1.5f);   // warm-up
    cudaEventRecord(e0);
    fns[kind]<<<blocks, PEAK_THREADS>>>(sink, iterations, 1.5f);
    cudaEventRecord(e1);
    int rc = cuda_status(cudaEventSynchronize(e1), "pipe benchmark");
    float ms = 0.0f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    if (rc) return rc;
    // lane-operations per inner statement: fma = 1 (x2 when packed), MUFU pair = 2, sub+add = 2
    const double per_stmt = (kind == 1) ? 2.0 : (kind == 0 ? 1.0 : 2.0);
    const double total    = per_stmt * 8.0 * PEAK_CHAINS * (double)iterations * (double)blocks * PEAK_THREADS;
    *ops_per_second       = total / (ms * 1e-3);
    if (milliseconds) *milliseconds = ms;
    return 0;
}
