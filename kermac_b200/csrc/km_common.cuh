// Shared device helpers for the kermac_b200 kernels (sm_100a only).
//
// The scalar math helpers restate the approximate-math conventions of the
// reference's include/kermac_internal_common.cuh:76-192 (sqrt.approx.ftz,
// ex2.approx.ftz(x * log2 e), ex2(p * lg2 v), copysign-based signum) so results
// agree with it to rounding.  The packed helpers use the sm_100-only f32x2
// instructions, which carry two fp32 lane-operations per issue slot.
#pragma once

#include <cstdint>
#include <cuda_runtime.h>

#include "../../include/kermac_b200.h"

namespace km {

typedef unsigned long long u64;

// ---------------------------------------------------------------- scalar math
__device__ __forceinline__ float sqrt_approx(float v) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float ex2_approx(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float lg2_approx(float v) {
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
// exp(v) as ex2(v * log2(e)); 0f3FB8AA3B is log2(e) rounded to fp32.
__device__ __forceinline__ float exp_approx(float v) {
    float t;
    asm("mul.ftz.f32 %0, %1, 0f3FB8AA3B;" : "=f"(t) : "f"(v));
    return ex2_approx(t);
}
// v^p for v >= 0 as ex2(p * lg2 v): pow(0, p>0) = 0, pow(0, 0) = NaN.
__device__ __forceinline__ float pow_approx(float v, float p) {
    float t = lg2_approx(v);
    asm("mul.ftz.f32 %0, %0, %1;" : "+f"(t) : "f"(p));
    return ex2_approx(t);
}

// ---------------------------------------------------------------- packed f32x2
__device__ __forceinline__ u64 pack2(float lo, float hi) {
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(u64 v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b) {
    u64 r;
    asm("sub.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 add2(u64 a, u64 b) {
    u64 r;
    asm("add.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b) {
    u64 r;
    asm("mul.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c) {
    u64 r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}

// ---------------------------------------------------------------- exp2 on the FP32 pipe
// The fractional-power inner step costs two MUFU operations per element (lg2, ex2)
// and the MUFU pipe has 16 lanes per SM against 128 FP32 lanes, so a kernel that
// sends both through MUFU is MUFU-bound with the FP32 pipe three quarters idle.
// ex2_poly2 evaluates 2^x for a packed pair on the FP32 pipe instead, so a share of
// the elements needs only one MUFU operation.
//
//   t     = x + (1.5 * 2^23 + 127)      round x to the nearest integer n; the low bits
//                                       of t then hold n + 127, the biased exponent
//   f     = x - (t - magic)             in [-0.5, 0.5]
//   r     = 2^f                         degree-5 polynomial, max relative error 2.9e-7
//                                       (ex2.approx is specified to 2 ulp = 2.4e-7)
//   scale = bits(t) << 23               2^n as a float
// The caller folds the scaling into its accumulate: acc = fma2(r, scale, acc).
// x is clamped to [-127, 128] first: at -127 (which is where lg2(0) * p = -inf lands)
// scale is exactly +0 and r exactly 1, so a zero difference still adds exactly 0; at
// 128 scale is +inf.  The clamps use the NaN-propagating min / max, so a NaN input
// still produces NaN (NaN * scale).
__device__ __forceinline__ float max_nan(float a, float b) {
    float r;
    asm("max.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ float min_nan(float a, float b) {
    float r;
    asm("min.NaN.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void ex2_poly2(float x0, float x1, u64& r, u64& scale) {
    x0 = min_nan(max_nan(x0, -127.0f), 128.0f);
    x1 = min_nan(max_nan(x1, -127.0f), 128.0f);
    const u64 x     = pack2(x0, x1);
    const u64 magic = pack2(12583039.0f, 12583039.0f);
    const u64 t     = add2(x, magic);
    const u64 f     = sub2(x, sub2(t, magic));
    // 2^f = 1 + f (c1 + f (c2 + f (c3 + f (c4 + f c5))))
    u64 q = fma2(f, pack2(1.3390867e-3f, 1.3390867e-3f), pack2(9.6663740e-3f, 9.6663740e-3f));
    q     = fma2(q, f, pack2(5.5503570e-2f, 5.5503570e-2f));
    q     = fma2(q, f, pack2(2.4022348e-1f, 2.4022348e-1f));
    q     = fma2(q, f, pack2(6.9314718e-1f, 6.9314718e-1f));
    r     = fma2(q, f, pack2(1.0f, 1.0f));
    float t0, t1;
    unpack2(t, t0, t1);
    scale = pack2(__int_as_float(__float_as_int(t0) << 23), __int_as_float(__float_as_int(t1) << 23));
}

// ---------------------------------------------------------------- result stores
// Ordinary stores, or multimem.st to an NVSwitch multicast address: one store that the
// switch delivers to the same offset of every GPU bound to the multicast object.
__device__ __forceinline__ void store_result4(float* dst, float v0, float v1, float v2, float v3, bool multicast) {
    if (multicast) {
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(dst), "f"(v0), "f"(v1),
                     "f"(v2), "f"(v3)
                     : "memory");
    } else {
        *reinterpret_cast<float4*>(dst) = make_float4(v0, v1, v2, v3);
    }
}
__device__ __forceinline__ void store_result1(float* dst, float v, bool multicast) {
    if (multicast) {
        asm volatile("multimem.st.relaxed.sys.global.f32 [%0], %1;" ::"l"(dst), "f"(v) : "memory");
    } else {
        *dst = v;
    }
}

// ---------------------------------------------------------------- async copies
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
// 16-byte global->shared copy that reads only `src_bytes` (0..16) bytes and
// zero-fills the rest of the destination.
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
// 4-byte global->shared copy; src_bytes 0 zero-fills.
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src, int src_bytes) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Reads a hyper-parameter for batch entry l.
__device__ __forceinline__ float read_hyper(const KmHyper& h, int l) {
    return h.ptr ? h.ptr[static_cast<long long>(l) * h.batch_stride] : h.value;
}

// The outer power, epsilon mask and kernel function applied to one accumulated
// sum, in the order of the reference's epilogue (include/build_a_kernel.cuh:374-427):
// outer power; values below epsilon become 0 (only when a kernel function is
// chosen); Laplace exp(-x / bw) or Gaussian exp(-x / (2 bw^2)).
struct Epilogue {
    int   outer_power;
    int   kernel_type;
    float p_outer;
    float neg_gamma;   // -1/bw (Laplace) or -1/(2 bw^2) (Gaussian)
    float epsilon;

    __device__ __forceinline__ float operator()(float acc) const {
        switch (outer_power) {
            case KM_POW_ABS: acc = fabsf(acc); break;
            case KM_POW_SQUARE: acc = acc * acc; break;
            case KM_POW_SQRT: acc = sqrt_approx(acc); break;
            case KM_POW_POW: acc = pow_approx(acc, p_outer); break;
            default: break;
        }
        if (kernel_type != KM_KERNEL_NONE) {
            if (acc < epsilon) acc = 0.0f;
            acc = exp_approx(acc * neg_gamma);
        }
        return acc;
    }
};

// The same chain with the outer power and the kernel function known at compile time.
template <int OP, int KT>
__device__ __forceinline__ float epilogue_value(const Epilogue& e, float acc) {
    if constexpr (OP == KM_POW_ABS) acc = fabsf(acc);
    else if constexpr (OP == KM_POW_SQUARE) acc = acc * acc;
    else if constexpr (OP == KM_POW_SQRT) acc = sqrt_approx(acc);
    else if constexpr (OP == KM_POW_POW) acc = pow_approx(acc, e.p_outer);
    if constexpr (KT != KM_KERNEL_NONE) {
        if (acc < e.epsilon) acc = 0.0f;
        acc = exp_approx(acc * e.neg_gamma);
    }
    return acc;
}

template <int OP, int KT>
__device__ __forceinline__ void epilogue_columns(const Epilogue& e, u64 (&acc)[8][4], int first, int count) {
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            if (i < first || i >= first + count) continue;
            float v0, v1;
            unpack2(acc[j][i], v0, v1);
            acc[j][i] = pack2(epilogue_value<OP, KT>(e, v0), epilogue_value<OP, KT>(e, v1));
        }
}

// Applies the chain in place to the packed columns [first, first + count) of a thread's
// 8 x 8 block.  The common chains get straight-line code (the choice is made once per
// call, not once per value); every other combination takes the generic path.  All paths
// compute the same values as Epilogue::operator().
__device__ __forceinline__ void apply_epilogue(const Epilogue& e, u64 (&acc)[8][4], int first, int count) {
    const int op = e.outer_power, kt = e.kernel_type;
    if (op == KM_POW_SQRT && kt == KM_KERNEL_LAPLACE) epilogue_columns<KM_POW_SQRT, KM_KERNEL_LAPLACE>(e, acc, first, count);
    else if (op == KM_POW_NOOP && kt == KM_KERNEL_LAPLACE) epilogue_columns<KM_POW_NOOP, KM_KERNEL_LAPLACE>(e, acc, first, count);
    else if (op == KM_POW_NOOP && kt == KM_KERNEL_GAUSSIAN) epilogue_columns<KM_POW_NOOP, KM_KERNEL_GAUSSIAN>(e, acc, first, count);
    else if (op == KM_POW_NOOP && kt == KM_KERNEL_NONE) { /* identity */ }
    else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (i < first || i >= first + count) continue;
                float v0, v1;
                unpack2(acc[j][i], v0, v1);
                acc[j][i] = pack2(e(v0), e(v1));
            }
    }
}

__device__ __forceinline__ Epilogue make_epilogue(int outer_power, int kernel_type, const KmHyper& p_outer,
                                                  const KmHyper& bandwidth, float epsilon, int l) {
    Epilogue e;
    e.outer_power = outer_power;
    e.kernel_type = kernel_type;
    e.p_outer     = (outer_power == KM_POW_POW) ? read_hyper(p_outer, l) : 0.0f;
    e.epsilon     = epsilon;
    e.neg_gamma   = 0.0f;
    if (kernel_type != KM_KERNEL_NONE) {
        float bw    = read_hyper(bandwidth, l);
        float gamma = (kernel_type == KM_KERNEL_LAPLACE) ? (1.0f / bw) : (1.0f / (2.0f * bw * bw));
        e.neg_gamma = -gamma;
    }
    return e;
}

// Inner-step identifiers: operator x power of the reference's template pair
// (InnerOperator, PowerType inner), include/build_a_kernel.cuh:344-366.
enum InnerId {
    IN_DIFF_ABS = 0,
    IN_DIFF_SQUARE,
    IN_DIFF_POW,
    IN_DIFF_NOOP,
    IN_DIFF_SQRT,
    IN_DOT_NOOP,
    IN_DOT_ABS,
    IN_DOT_SQUARE,
    IN_DOT_SQRT,
    IN_DOT_POW,
    IN_COUNT
};

__host__ __device__ inline int inner_id(int op, int power) {
    if (op == KM_INNER_DIFF) {
        switch (power) {
            case KM_POW_ABS: return IN_DIFF_ABS;
            case KM_POW_SQUARE: return IN_DIFF_SQUARE;
            case KM_POW_POW: return IN_DIFF_POW;
            case KM_POW_NOOP: return IN_DIFF_NOOP;
            case KM_POW_SQRT: return IN_DIFF_SQRT;
        }
    } else if (op == KM_INNER_DOT) {
        switch (power) {
            case KM_POW_NOOP: return IN_DOT_NOOP;
            case KM_POW_ABS: return IN_DOT_ABS;
            case KM_POW_SQUARE: return IN_DOT_SQUARE;
            case KM_POW_SQRT: return IN_DOT_SQRT;
            case KM_POW_POW: return IN_DOT_POW;
        }
    }
    return -1;
}

// Which of the 8 x 4 element pairs of a register block take their exponential on the FP32
// pipe (ex2_poly2) rather than on MUFU: KM_POW_POLY_EIGHTHS of every 8 pairs.
#ifndef KM_POW_POLY_EIGHTHS
#define KM_POW_POLY_EIGHTHS 6
#endif
__device__ __forceinline__ constexpr bool pow_pair_uses_fp32_exp(int n, int mp) {
    return ((n & 1) * 4 + mp) < KM_POW_POLY_EIGHTHS;
}

// One k step of an 8 (rows of the pair-packed operand) x 8 register block.
//   ap[4]  : the 8 values of the m-side operand as 4 packed pairs (m, m+1)
//   bv[8]  : the 8 values of the n-side operand
//   acc    : acc[n][mp] packed pair of accumulators for (m = 2 mp, 2 mp + 1)
// `sgn` is +1 normally and -1 when the launcher exchanged the two operands (so
// that signed inner steps still see b - a).
template <int INNER>
__device__ __forceinline__ void inner_block(u64 (&acc)[8][4], const u64 (&ap)[4], const float (&bv)[8], float p_inner,
                                            float sgn) {
#pragma unroll
    for (int n = 0; n < 8; ++n) {
        const u64 bd = pack2(bv[n], bv[n]);
#pragma unroll
        for (int mp = 0; mp < 4; ++mp) {
            if constexpr (INNER == IN_DIFF_SQUARE) {
                const u64 d = sub2(bd, ap[mp]);
                acc[n][mp]  = fma2(d, d, acc[n][mp]);
            } else if constexpr (INNER == IN_DOT_NOOP) {
                acc[n][mp] = fma2(bd, ap[mp], acc[n][mp]);
            } else {
                const u64 d = (INNER >= IN_DOT_NOOP) ? mul2(bd, ap[mp]) : sub2(bd, ap[mp]);
                float d0, d1, a0, a1;
                unpack2(d, d0, d1);
                unpack2(acc[n][mp], a0, a1);
                if constexpr (INNER == IN_DIFF_ABS || INNER == IN_DOT_ABS) {
                    a0 += fabsf(d0);
                    a1 += fabsf(d1);
                } else if constexpr (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) {
                    if (pow_pair_uses_fp32_exp(n, mp)) {
                        // most pairs: lg2 on MUFU, the exponential on the FP32 pipe.  A pair costs
                        // ~30 issue slots this way against ~10 (and 32 MUFU cycles instead of 16)
                        // the all-MUFU way; the share is set where the kernel measured fastest.
                        const u64 x = mul2(pack2(lg2_approx(fabsf(d0)), lg2_approx(fabsf(d1))), pack2(p_inner, p_inner));
                        float x0, x1;
                        unpack2(x, x0, x1);
                        u64 r, scale;
                        ex2_poly2(x0, x1, r, scale);
                        acc[n][mp] = fma2(r, scale, acc[n][mp]);
                        continue;
                    }
                    a0 += pow_approx(fabsf(d0), p_inner);
                    a1 += pow_approx(fabsf(d1), p_inner);
                } else if constexpr (INNER == IN_DIFF_NOOP) {
                    a0 += d0;
                    a1 += d1;
                } else if constexpr (INNER == IN_DIFF_SQRT) {
                    a0 += sqrt_approx(d0 * sgn);
                    a1 += sqrt_approx(d1 * sgn);
                } else if constexpr (INNER == IN_DOT_SQUARE) {
                    a0 = fmaf(d0, d0, a0);
                    a1 = fmaf(d1, d1, a1);
                } else if constexpr (INNER == IN_DOT_SQRT) {
                    a0 += sqrt_approx(d0);
                    a1 += sqrt_approx(d1);
                }
                acc[n][mp] = pack2(a0, a1);
            }
        }
    }
}

// Consumes one staged k slab ([BK][PITCH] floats per operand, tile dimension
// contiguous) for a thread whose 8 x 8 block reads the m-side at sa + {0, 32} and
// the n-side at sb + {0, 16}.  Only the first `kvalid` k rows are used, so a partial
// last slab contributes exactly the rows that exist.
template <int INNER, int BK, int PITCH>
__device__ __forceinline__ void consume_slab(u64 (&acc)[8][4], const float* sa, const float* sb, int kvalid,
                                             float p_inner, float sgn) {
    auto step = [&](int kk) {
        const ulonglong2 a0 = *reinterpret_cast<const ulonglong2*>(sa + kk * PITCH);
        const ulonglong2 a1 = *reinterpret_cast<const ulonglong2*>(sa + kk * PITCH + 32);
        const u64   ap[4] = {a0.x, a0.y, a1.x, a1.y};
        float bv[8];
        if constexpr (INNER == IN_DIFF_ABS || INNER == IN_DOT_ABS) {
            // The |.| step reads the n-side values one by one (warp-wide broadcasts): each lands in the
            // low half of the register pair it is duplicated into, which measured 0.8 % faster here
            // (59.6 against 60.1 ms at 30000 x 30000 x 1024); the other steps measured no difference.
#pragma unroll
            for (int n = 0; n < 8; ++n) bv[n] = sb[kk * PITCH + (n >> 2) * 16 + (n & 3)];
        } else {
            const float4 b0 = *reinterpret_cast<const float4*>(sb + kk * PITCH);
            const float4 b1 = *reinterpret_cast<const float4*>(sb + kk * PITCH + 16);
            bv[0] = b0.x; bv[1] = b0.y; bv[2] = b0.z; bv[3] = b0.w;
            bv[4] = b1.x; bv[5] = b1.y; bv[6] = b1.z; bv[7] = b1.w;
        }
        inner_block<INNER>(acc, ap, bv, p_inner, sgn);
    };
    // The whole slab is unrolled, so operand loads are scheduled ahead of the math across all
    // of its rows.  The fractional-power step is ~30 instructions per element; unrolling it
    // that far would not fit the instruction cache, so it is unrolled by 2 only.
    constexpr int UNROLL = (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) ? 2 : BK;
    if (kvalid >= BK) {
#pragma unroll UNROLL
        for (int kk = 0; kk < BK; ++kk) step(kk);
    } else {
#pragma unroll 1
        for (int kk = 0; kk < kvalid; ++kk) step(kk);
    }
}

}  // namespace km
