// Register-only microbenchmarks of the arithmetic pipes the distance kernels are
// bound by.  They give the roofline denominators (fp32 lane-operations per second,
// MUFU operations per second) for the device and clock the benchmark actually
// runs at, instead of a nominal figure.
#include "km_build_params.cuh"
#include "km_host.h"
#include "km_mbar.cuh"
#include "km_tcgen05.cuh"

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

// The product inner loop (consume_slab: 128-bit shared loads, duplicate moves, packed
// sub / fma or sub / add|.|) running from a shared-memory slab that is filled once, with
// no global staging, barriers or epilogue: the ceiling the instruction mix itself allows.
template <int INNER>
__global__ void __launch_bounds__(256, 2) inner_loop_kernel(float* sink, int slabs, float seed) {
    constexpr int BK = BUILD_CPA_BK, PITCH = BUILD_CPA_PITCH;
    __shared__ __align__(16) float sa[BK * PITCH];
    __shared__ __align__(16) float sb[BK * PITCH];
    for (int i = threadIdx.x; i < BK * PITCH; i += 256) {
        sa[i] = seed + 1e-3f * i;
        sb[i] = seed - 2e-3f * i;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* pa = sa + (warp & 1) * 64 + (lane & 7) * 4;
    const float* pb = sb + (warp >> 1) * 32 + (lane >> 3) * 4;
    u64 acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0ull;
    for (int s = 0; s < slabs; ++s) {
        // alternate the start row (0 or 4; rows shift .. shift + BK - 5 stay inside the BK-row
        // slab) so the loads are not loop invariant
        const int shift = (s & 1) * 4;
        consume_slab<INNER, BK - 4, PITCH>(acc, pa + shift * PITCH, pb + shift * PITCH, BK, 1.3f, 1.0f);
    }
    float t = 0.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float lo, hi;
            unpack2(acc[j][i], lo, hi);
            t += lo + hi;
        }
    if (t == 123.456f) sink[0] = t;
}

// The gradient's k step for a 4 (m) x 4 (n) x 4 (channel) thread block in registers only:
// per (n, m-pair) one packed subtract, the sign flip (two bit operations) and four channel
// FMAs whose three sources are three different registers (coefficient, weight, accumulator).
// PACKED: the FMAs as fma.rn.f32x2 on register pairs; otherwise as two scalar FMAs each.
// Nothing is loop invariant (the n-side operand changes every step), so the count of
// instructions per step is the kernel's, without loads, staging or barriers.
template <bool PACKED>
__global__ void __launch_bounds__(256, 2) grad_step_kernel(float* sink, int steps, float seed) {
    u64   dv[4][2], av[2], acc[4][4][2];
    float cv[4], bv[4], accs[4][4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        bv[j] = seed * (j + 1) + threadIdx.x;
#pragma unroll
        for (int h = 0; h < 2; ++h) dv[j][h] = pack2(seed + j + 0.25f * h, seed - j + 0.5f * threadIdx.x);
#pragma unroll
        for (int o = 0; o < 4; ++o) {
            acc[j][o][0] = acc[j][o][1] = 0ull;
#pragma unroll
            for (int e = 0; e < 4; ++e) accs[j][o][e] = 0.0f;
        }
    }
    av[0] = pack2(seed, seed + 1.0f);
    av[1] = pack2(seed + 2.0f, seed + 3.0f);
#pragma unroll
    for (int o = 0; o < 4; ++o) cv[o] = 0.5f + o + 1e-3f * threadIdx.x;
    for (int it = 0; it < steps; ++it) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            u64 cd[4];
#pragma unroll
            for (int o = 0; o < 4; ++o) cd[o] = pack2(cv[o], cv[o]);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                bv[j]        = __int_as_float(__float_as_int(bv[j]) ^ (it + r));   // stands in for the operand load
                const u64 bd = pack2(bv[j], bv[j]);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const u64 diff = sub2(dv[j][h], bd);
                    const u64 w    = av[h] ^ (diff & 0x8000000080000000ull);
                    if constexpr (PACKED) {
#pragma unroll
                        for (int o = 0; o < 4; ++o) acc[j][o][h] = fma2(cd[o], w, acc[j][o][h]);
                    } else {
                        float w0, w1;
                        unpack2(w, w0, w1);
#pragma unroll
                        for (int o = 0; o < 4; ++o) {
                            accs[j][o][2 * h]     = fmaf(cv[o], w0, accs[j][o][2 * h]);
                            accs[j][o][2 * h + 1] = fmaf(cv[o], w1, accs[j][o][2 * h + 1]);
                        }
                    }
                }
            }
        }
    }
    float t = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int o = 0; o < 4; ++o) {
            float a0, a1, a2, a3;
            unpack2(acc[j][o][0], a0, a1);
            unpack2(acc[j][o][1], a2, a3);
            t += a0 + a1 + a2 + a3 + accs[j][o][0] + accs[j][o][1] + accs[j][o][2] + accs[j][o][3];
        }
    if (t == 123.456f) sink[0] = t;
}

typedef void (*PipeFn)(float*, int, float);

// Issue rate of the narrow MMAs of the tensor-core gradient kernel: one thread per SM issues
// tcgen05.mma kind::tf32, 128 rows x N columns x 8 k, A operand from tensor memory, B from shared
// memory, all into one accumulator (the pipe does not wait on a dependent accumulate).  Operand values
// are whatever the memories hold; only the time matters.  The wait for the last MMA is bounded.
template <int N>
__global__ void __launch_bounds__(128) mma_rate_kernel(float* sink, int steps, float) {
    __shared__ __align__(1024) unsigned char b_tile[256 * 128];
    __shared__ __align__(8) unsigned long long s_bar;
    __shared__ uint32_t s_tmem;
    for (int i = threadIdx.x; i < 256 * 128 / 4; i += blockDim.x) reinterpret_cast<float*>(b_tile)[i] = 0.0f;
    const uint32_t bar = smem_u32(&s_bar);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < 32) tc::tmem_alloc(smem_u32(&s_tmem), 512);
    tc::fence_smem_to_async();
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem = s_tmem;
    if (threadIdx.x == 0) {
        constexpr uint32_t idesc = tc::instr_desc_tf32(128, N);
        const uint64_t db        = tc::smem_desc_k_major_sw128(smem_u32(b_tile));
        for (int it = 0; it < steps; ++it) {
#pragma unroll
            for (int j = 0; j < 8; ++j) tc::mma_tf32_a_tmem(tmem + 256, tmem + j * 8, db, idesc, true);
        }
        tc::commit(bar);
        if (!mbar_wait_bounded(bar, 0)) sink[1] = 1.0f;
    }
    tc::fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) tc::tmem_dealloc(tmem, 512);
}

}  // namespace
}  // namespace km

extern "C" int kermac_b200_measure_pipe(int32_t kind, int32_t iterations, double* ops_per_second,
                                        double* milliseconds) {
    using namespace km;
    if (!ops_per_second) return fail(KM_ERR_NULL_POINTER, "ops_per_second is NULL");
    if (kind < 0 || kind > 11) return fail(KM_ERR_BAD_ENUM, "kind %d is not a pipe benchmark", kind);
    if (iterations < 1 || iterations > (1 << 24)) return fail(KM_ERR_BAD_SHAPE, "iterations out of range");
    if (int rc = require_sm100()) return rc;
    PipeFn fns[12] = {pipe_kernel<0>, pipe_kernel<1>, pipe_kernel<2>, pipe_kernel<3>,
                      inner_loop_kernel<IN_DIFF_SQUARE>, inner_loop_kernel<IN_DIFF_ABS>,
                      grad_step_kernel<true>, grad_step_kernel<false>,
                      mma_rate_kernel<32>, mma_rate_kernel<64>, mma_rate_kernel<128>, mma_rate_kernel<256>};
    float* sink   = nullptr;
    if (int rc = cuda_status(cudaMalloc(&sink, 256), "cudaMalloc")) return rc;
    const bool mma   = kind >= 8;
    const int blocks = sm_count() * (mma ? 1 : (kind >= 4 ? 2 : 8));
    const int threads = mma ? 128 : PEAK_THREADS;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    fns[kind]<<<blocks, threads>>>(sink, iterations / 8 + 1, 1.5f);   // warm-up
    cudaEventRecord(e0);
    fns[kind]<<<blocks, threads>>>(sink, iterations, 1.5f);
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
    double total          = per_stmt * 8.0 * PEAK_CHAINS * (double)iterations * (double)blocks * PEAK_THREADS;
    // inner-loop kinds: `iterations` slabs of BK - 4 k rows, 64 element-steps per thread and row, 2 lane-ops each
    if (kind >= 4) total = 2.0 * 64.0 * (BUILD_CPA_BK - 4) * (double)iterations * (double)blocks * PEAK_THREADS;
    // gradient-step kinds: 4 steps per iteration, 16 (m, n) pairs per thread and step, 1 + 4 lane-ops each
    if (kind >= 6) total = 4.0 * 16.0 * 5.0 * (double)iterations * (double)blocks * PEAK_THREADS;
    // MMA kinds: 8 MMAs per iteration and SM
    if (mma) total = 8.0 * (double)iterations * (double)blocks;
    *ops_per_second       = total / (ms * 1e-3);
    if (milliseconds) *milliseconds = ms;
    return 0;
}
