// kermac_b200_cdist_grad: the p-norm gradient contraction
//   out[l, o, n, m] = sum_k c[l, o, k] * a[l, k, m] * g(d[l, n, m] - b[l, n, k])
// restating what the reference's kernel_cute_p_norm_kernel_gradient computes
// (include/p_norm_gradient.cuh:22-405) with a different work decomposition:
//   - a thread block owns a 64 (m) x TN (n) tile for up to OT output channels, with
//     OT chosen from {1, 2, 4, 8, 16} to fit O (the reference always spends 32);
//   - the weight w = a * g(diff) is formed once per (m, n, k) and reused for every
//     channel; for p = 1 the sign is applied with one bit operation on a;
//   - differences, weights and channel FMAs run on packed pairs along m;
//   - the contracted k range can be split over several thread blocks, whose partial
//     tiles go to caller-provided scratch and are summed in a fixed order by a
//     second kernel, so results do not depend on scheduling.  The split is chosen so
//     that the thread blocks fill whole waves of the machine (two blocks per SM);
//   - blocks that share a tile of the weight matrix a (the n-tiles of one m-column and
//     k range) are neighbours in launch order, so a is read from DRAM once;
//   - p = 1.5 takes |x|^(p-1) as one sqrt.approx instead of the lg2 / ex2 pair.
#include <mutex>

#include "km_common.cuh"
#include "km_host.h"

namespace km {
namespace {

constexpr int G_THREADS = 256;
constexpr int G_TM      = 64;
constexpr int G_BK      = 32;   // k rows per staged slab (a multiple of 8)
constexpr int G_STAGES  = 3;
constexpr int G_UNROLL  = 32;   // k rows of a slab unrolled together
// Kernel-side norm kinds: the three of the C-ABI plus the square-root form of KM_NORM_P
// for p - 1 == 0.5, chosen by the launcher when p is a host scalar.
constexpr int G_NORM_SQRT = 3;
static_assert(G_NORM_SQRT == GT_NORM_SQRT && G_BK == GT_BK, "the two gradient kernels share the planner");
// Channels from which KM_CONTRACT_AUTO takes the tensor-core kernel.
constexpr int KM_GRAD_TENSOR_MIN_O = 17;

struct GradParams {
    int M, N, O, K, L;
    const float* A; long long lda, a_sl;
    const float* B; long long ldb, b_sl;
    const float* C; long long ldc, c_sl;
    const float* D; long long ldd, d_sl;
    float*       E; long long e_sn, e_so, e_sl;   // destination (out, or scratch when split)
    KmHyper p;
    int tiles_m, tiles_n, o_chunks, splits;
    int k_per_split;                                // multiple of G_BK
    long long split_stride;                         // elements between partial results of consecutive splits
    int a_vec, e_vec;
};

__device__ __forceinline__ u64 flip_sign2(u64 a, u64 diff) {
    // a with the sign bit of diff xor-ed in, lane-wise: copysign(1, diff) * a
    return a ^ (diff & 0x8000000080000000ull);
}

// Thread blocks resident per SM that every tile shape is compiled for.
constexpr int grad_min_blocks(int, int) { return 2; }

template <int NORM, int OT, int NT>
__global__ void __launch_bounds__(G_THREADS, grad_min_blocks(OT, NT)) grad_kernel(const __grid_constant__ GradParams p) {
    constexpr int TN      = 16 * NT;
    constexpr int PITCH_A = G_TM + 4;
    constexpr int PITCH_B = TN + 4;
    constexpr int PITCH_C = (OT < 4 ? 4 : OT);
    constexpr int STAGE_FLOATS = G_BK * (PITCH_A + PITCH_B + PITCH_C);
    extern __shared__ __align__(16) float smem[];      // G_STAGES * STAGE_FLOATS floats (grad_smem_bytes)

    const int tid = threadIdx.x;
    const int tmi = tid & 15, tni = tid >> 4;

    // n-tiles fastest: the blocks that read the same (k range, m-column) tile of a run together
    int bx          = blockIdx.x;
    const int tn    = bx % p.tiles_n; bx /= p.tiles_n;
    const int split = bx % p.splits;  bx /= p.splits;
    const int tm    = bx;
    const int oc    = blockIdx.y;
    const int l     = blockIdx.z;
    const int m0 = tm * G_TM, n0 = tn * TN, o0 = oc * OT;

    const int k_begin = split * p.k_per_split;
    const int k_end   = min(p.K, k_begin + p.k_per_split);
    const int ktiles  = (k_end > k_begin) ? (k_end - k_begin + G_BK - 1) / G_BK : 0;

    const float* A = p.A + (long long)l * p.a_sl + m0;
    const float* B = p.B + (long long)l * p.b_sl + (long long)n0 * p.ldb;
    const float* C = p.C + (long long)l * p.c_sl + (long long)o0 * p.ldc;
    const float* D = p.D + (long long)l * p.d_sl;

    float pm1 = 0.0f;
    if (NORM == KM_NORM_P) pm1 = read_hyper(p.p, l) - 1.0f;

    // d values of this thread: rows n0 + tni * NT + j, columns m0 + tmi * 4 + {0..3}
    u64 dv[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int n = n0 + tni * NT + j;
        float v[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int m = m0 + tmi * 4 + e;
            v[e]        = (n < p.N && m < p.M) ? D[(long long)n * p.ldd + m] : 0.0f;
        }
        dv[j][0] = pack2(v[0], v[1]);
        dv[j][1] = pack2(v[2], v[3]);
    }

    u64 acc[NT][OT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j)
#pragma unroll
        for (int o = 0; o < OT; ++o) acc[j][o][0] = acc[j][o][1] = 0ull;

    auto stage = [&](int s, int kt) {
        float* sa = smem + s * STAGE_FLOATS;
        float* sb = sa + G_BK * PITCH_A;
        float* sc = sb + G_BK * PITCH_B;
        const int k0 = k_begin + kt * G_BK;
        if (p.a_vec) {
            // G_BK k rows x 16 chunks of 4 m
#pragma unroll
            for (int i = 0; i < (G_BK * G_TM / 4) / G_THREADS; ++i) {
                const int idx = tid + i * G_THREADS;
                const int kk = idx >> 4, t = (idx & 15) << 2, gk = k0 + kk;
                int valid = min(4, p.M - m0 - t);
                valid     = (gk < k_end && valid > 0) ? valid : 0;
                cp_async_16(smem_u32(sa + kk * PITCH_A + t), valid ? A + (long long)gk * p.lda + t : p.A, valid * 4);
            }
        } else {
#pragma unroll
            for (int i = 0; i < (G_BK * G_TM) / G_THREADS; ++i) {
                const int idx = tid + i * G_THREADS;
                const int t = idx & (G_TM - 1), kk = idx >> 6, gk = k0 + kk;
                const bool ok = gk < k_end && (m0 + t) < p.M;
                cp_async_4(smem_u32(sa + kk * PITCH_A + t), ok ? A + (long long)gk * p.lda + t : p.A, ok ? 4 : 0);
            }
        }
        // b and c are k-contiguous in global memory and staged k-major.  A warp copies 8
        // consecutive k of 4 rows: 32-byte runs on the global side, and on the shared side
        // banks 4 kk + t (pitches are 4 mod 32 or 20), all different, so the 4-byte writes
        // do not collide.
        constexpr int K8 = G_BK / 8;
#pragma unroll
        for (int i = 0; i < (G_BK * TN + G_THREADS - 1) / G_THREADS; ++i) {
            const int idx = tid + i * G_THREADS;
            if (idx < G_BK * TN) {
                const int kk = (idx & 7) + ((idx >> 5) % K8) * 8;
                const int t  = ((idx >> 3) & 3) + (idx / (32 * K8)) * 4;
                const int gk = k0 + kk;
                const bool ok = gk < k_end && (n0 + t) < p.N;
                cp_async_4(smem_u32(sb + kk * PITCH_B + t), ok ? B + (long long)t * p.ldb + gk : p.B, ok ? 4 : 0);
            }
        }
        constexpr int C_ROWS = (OT < 4 ? 4 : OT);
#pragma unroll
        for (int i = 0; i < (G_BK * C_ROWS + G_THREADS - 1) / G_THREADS; ++i) {
            const int idx = tid + i * G_THREADS;
            if (idx < G_BK * C_ROWS) {
                const int kk = (idx & 7) + ((idx >> 5) % K8) * 8;
                const int t  = ((idx >> 3) & 3) + (idx / (32 * K8)) * 4;
                const int gk = k0 + kk;
                const bool ok = gk < k_end && (o0 + t) < p.O;
                if (t < OT) cp_async_4(smem_u32(sc + kk * PITCH_C + t), ok ? C + (long long)t * p.ldc + gk : p.C, ok ? 4 : 0);
            }
        }
    };

    auto step = [&](const float* sa, const float* sb, const float* sc, int kk) {
        const ulonglong2 a4 = *reinterpret_cast<const ulonglong2*>(sa + kk * PITCH_A + tmi * 4);
        const u64 av[2]     = {a4.x, a4.y};
        // b and c rows of this k: 128-bit shared loads where the tile shape allows
        float bv[NT];
        if constexpr (NT == 4) {
            const float4 b4 = *reinterpret_cast<const float4*>(sb + kk * PITCH_B + tni * 4);
            bv[0] = b4.x; bv[1] = b4.y; bv[2] = b4.z; bv[3] = b4.w;
        } else if constexpr (NT == 2) {
            const float2 b2 = *reinterpret_cast<const float2*>(sb + kk * PITCH_B + tni * 2);
            bv[0] = b2.x; bv[1] = b2.y;
        } else {
            bv[0] = sb[kk * PITCH_B + tni];
        }
        float cv[OT];
        if constexpr (OT >= 4) {
#pragma unroll
            for (int o = 0; o < OT; o += 4) {
                const float4 c4 = *reinterpret_cast<const float4*>(sc + kk * PITCH_C + o);
                cv[o] = c4.x; cv[o + 1] = c4.y; cv[o + 2] = c4.z; cv[o + 3] = c4.w;
            }
        } else {
#pragma unroll
            for (int o = 0; o < OT; ++o) cv[o] = sc[kk * PITCH_C + o];
        }
        u64 cd[OT];
#pragma unroll
        for (int o = 0; o < OT; ++o) cd[o] = pack2(cv[o], cv[o]);
        // Order of the 8 (n, m-pair) x OT channel FMAs of a k row.  They all cost the same in theory;
        // in practice the order decides which source operands repeat from one instruction to the next
        // and how the compiler lays the registers out, and a few per cent hang on it.  Measured at
        // K = 30000, M = 4096, N = 256, O = 4 (ms, orders: 0 = weight by weight as it is computed, then
        // with all weights of the row first, 1 = channel / n / pair, 3 = pair / channel / n):
        //   p = 1:   0: 6.45   1: 6.24   3: 6.39        p = 2:   0: 6.37   1: 6.25   3: 6.21
        //   p = 1.5: 0: 8.72   1: 8.82   3: 8.66        p = 1.7: 0: 14.84  1: 15.78  3: 15.06
        // With the two multiplicands exchanged (weight first, coefficient second) order 1 falls back to 6.9 ms:
        // what pays is the FIRST source repeating over a long run of instructions (the coefficient pair over
        // all 8 weights of the row).  Other channel tiles measured no difference and keep order 0.
        constexpr int ORDER = (OT != 4) ? 0 : (NORM == KM_NORM_L1 ? 1 : ((NORM == KM_NORM_L2 || NORM == G_NORM_SQRT) ? 3 : 0));
        if constexpr (ORDER == 0) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
            const u64 bd = pack2(bv[j], bv[j]);
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const u64 diff = sub2(dv[j][h], bd);
                u64 w;
                if constexpr (NORM == KM_NORM_L1) {
                    w = flip_sign2(av[h], diff);
                } else if constexpr (NORM == KM_NORM_L2) {
                    w = mul2(av[h], diff);
                } else if constexpr (NORM == G_NORM_SQRT) {
                    // |x|^(1/2) sign(x): one MUFU operation per element instead of two
                    float d0, d1;
                    unpack2(diff, d0, d1);
                    w = flip_sign2(mul2(av[h], pack2(sqrt_approx(fabsf(d0)), sqrt_approx(fabsf(d1)))), diff);
                } else {
                    float d0, d1;
                    unpack2(diff, d0, d1);
                    if (h == 0 && (j & 1) == 0 && NT > 1) {
                        // one pair in four takes only lg2 on MUFU and the exponential on the
                        // FP32 pipe (ex2_poly2); more than that and instruction issue, not MUFU,
                        // becomes the limit
                        const u64 x = mul2(pack2(lg2_approx(fabsf(d0)), lg2_approx(fabsf(d1))), pack2(pm1, pm1));
                        float x0, x1;
                        unpack2(x, x0, x1);
                        u64 r, scale;
                        ex2_poly2(x0, x1, r, scale);
                        w = mul2(av[h], flip_sign2(mul2(r, scale), diff));
                    } else {
                        const float g0 = copysignf(pow_approx(fabsf(d0), pm1), d0);
                        const float g1 = copysignf(pow_approx(fabsf(d1), pm1), d1);
                        w              = mul2(av[h], pack2(g0, g1));
                    }
                }
#pragma unroll
                // A packed FMA whose three sources are three different register pairs (coefficient,
                // weight, accumulator) holds the FP32 pipe for about three cycles instead of two, which
                // is what bounds this loop (32 of them and 8 packed subtracts per k row: ~112 cycles for
                // 80 cycles of arithmetic).  Scalar FMAs (two per pair) and a half packed / half scalar
                // mix both measured slower: 7.5 and 7.0 ms against 6.6.
                for (int o = 0; o < OT; ++o) acc[j][o][h] = fma2(cd[o], w, acc[j][o][h]);
            }
        }
        } else {
            u64 wv[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const u64 bd = pack2(bv[j], bv[j]);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                const u64 diff = sub2(dv[j][h], bd);
                u64 w;
                if constexpr (NORM == KM_NORM_L1) {
                    w = flip_sign2(av[h], diff);
                } else if constexpr (NORM == KM_NORM_L2) {
                    w = mul2(av[h], diff);
                } else if constexpr (NORM == G_NORM_SQRT) {
                    // |x|^(1/2) sign(x): one MUFU operation per element instead of two
                    float d0, d1;
                    unpack2(diff, d0, d1);
                    w = flip_sign2(mul2(av[h], pack2(sqrt_approx(fabsf(d0)), sqrt_approx(fabsf(d1)))), diff);
                } else {
                    float d0, d1;
                    unpack2(diff, d0, d1);
                    if (h == 0 && (j & 1) == 0 && NT > 1) {
                        // one pair in four takes only lg2 on MUFU and the exponential on the
                        // FP32 pipe (ex2_poly2); more than that and instruction issue, not MUFU,
                        // becomes the limit
                        const u64 x = mul2(pack2(lg2_approx(fabsf(d0)), lg2_approx(fabsf(d1))), pack2(pm1, pm1));
                        float x0, x1;
                        unpack2(x, x0, x1);
                        u64 r, scale;
                        ex2_poly2(x0, x1, r, scale);
                        w = mul2(av[h], flip_sign2(mul2(r, scale), diff));
                    } else {
                        const float g0 = copysignf(pow_approx(fabsf(d0), pm1), d0);
                        const float g1 = copysignf(pow_approx(fabsf(d1), pm1), d1);
                        w              = mul2(av[h], pack2(g0, g1));
                    }
                }
                    wv[j][h] = w;
                }
            }
            if constexpr (ORDER == 1) {
#pragma unroll
                for (int o = 0; o < OT; ++o)
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int h = 0; h < 2; ++h) acc[j][o][h] = fma2(cd[o], wv[j][h], acc[j][o][h]);
            } else {
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int o = 0; o < OT; ++o)
#pragma unroll
                        for (int j = 0; j < NT; ++j) acc[j][o][h] = fma2(cd[o], wv[j][h], acc[j][o][h]);
            }
        }
    };

#pragma unroll
    for (int s = 0; s < G_STAGES - 1; ++s) {
        if (s < ktiles) stage(s, s);
        cp_async_commit();
    }
    for (int kt = 0; kt < ktiles; ++kt) {
        cp_async_wait<G_STAGES - 2>();
        __syncthreads();
        const int nk = kt + G_STAGES - 1;
        if (nk < ktiles) stage(nk % G_STAGES, nk);
        cp_async_commit();
        const float* sa = smem + (kt % G_STAGES) * STAGE_FLOATS;
        const float* sb = sa + G_BK * PITCH_A;
        const float* sc = sb + G_BK * PITCH_B;
        const int kvalid = k_end - (k_begin + kt * G_BK);
        if (kvalid >= G_BK) {
            // The whole 32-row slab unrolled measured fastest (6.45 ms against 6.58 with 16-row slabs
            // and 6.65 with an unroll of 8 at K = 30000, M = 4096, N = 256, O = 4); the handful of
            // registers that spill are reloaded about four times per slab, not per k row.
#pragma unroll G_UNROLL
            for (int kk = 0; kk < G_BK; ++kk) step(sa, sb, sc, kk);
        } else {
#pragma unroll 1
            for (int kk = 0; kk < kvalid; ++kk) step(sa, sb, sc, kk);
        }
    }
    cp_async_wait<0>();

    float* E = p.E + (long long)split * p.split_stride + (long long)l * p.e_sl;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int n = n0 + tni * NT + j;
        if (n >= p.N) continue;
#pragma unroll
        for (int o = 0; o < OT; ++o) {
            if (o0 + o >= p.O) continue;
            float* row = E + (long long)(o0 + o) * p.e_so + (long long)n * p.e_sn;
            const int m = m0 + tmi * 4;
            float v[4];
            unpack2(acc[j][o][0], v[0], v[1]);
            unpack2(acc[j][o][1], v[2], v[3]);
            if (p.e_vec && m + 3 < p.M) {
                *reinterpret_cast<float4*>(row + m) = make_float4(v[0], v[1], v[2], v[3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (m + e < p.M) row[m + e] = v[e];
            }
        }
    }
}

// out[l][o][n][m] = sum over splits of partial[split][l][o][n][m] (dense partials).
__global__ void __launch_bounds__(256) grad_reduce_kernel(const float* __restrict__ partial, float* __restrict__ out,
                                                          int M, int N, int O, int L, int splits, long long split_stride,
                                                          long long o_sn, long long o_so, long long o_sl) {
    const long long total = (long long)L * O * N * M;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int sp = 0; sp < splits; ++sp) s += partial[sp * split_stride + i];
        long long r = i;
        const int m = (int)(r % M); r /= M;
        const int n = (int)(r % N); r /= N;
        const int o = (int)(r % O); r /= O;
        const int l = (int)r;
        out[l * o_sl + o * o_so + n * o_sn + m] = s;
    }
}

typedef void (*GradFn)(const GradParams);

struct GradChoice {
    GradFn fn;
    int    smem_bytes;
};

constexpr int grad_smem_bytes(int ot, int nt) {
    return G_STAGES * G_BK * ((G_TM + 4) + (16 * nt + 4) + (ot < 4 ? 4 : ot)) * 4;
}

template <int NORM>
GradChoice grad_fn_for(int ot) {
    switch (ot) {
        case 1: return {grad_kernel<NORM, 1, 4>, grad_smem_bytes(1, 4)};
        case 2: return {grad_kernel<NORM, 2, 4>, grad_smem_bytes(2, 4)};
        case 4: return {grad_kernel<NORM, 4, 4>, grad_smem_bytes(4, 4)};
        case 8: return {grad_kernel<NORM, 8, 2>, grad_smem_bytes(8, 2)};
        default: return {grad_kernel<NORM, 16, 1>, grad_smem_bytes(16, 1)};
    }
}
int nt_for(int ot) { return ot <= 4 ? 4 : (ot == 8 ? 2 : 1); }

struct GradPlan {
    GradParams p;
    int ot, nt;
    bool tensor;               // channel contraction on the tensor cores (km_grad_tensor.cu)
    int splits_wanted;
    long long partial_elems;   // elements of one dense partial result
};

int make_grad_plan(const KmGradArgs* a, GradPlan* plan) {
    if (!a) return fail(KM_ERR_NULL_POINTER, "args is NULL");
    if (a->m < 0 || a->n < 0 || a->o < 0 || a->k < 0 || a->l < 1)
        return fail(KM_ERR_BAD_SHAPE, "bad extents m=%d n=%d o=%d k=%d l=%d", a->m, a->n, a->o, a->k, a->l);
    if (a->l > 65535) return fail(KM_ERR_TOO_LARGE, "at most 65535 batch entries per call");
    const bool empty = (a->m == 0 || a->n == 0 || a->o == 0);
    if (!empty && (!a->out || !a->d || (a->k > 0 && (!a->a || !a->b || !a->c))))
        return fail(KM_ERR_NULL_POINTER, "a, b, c, d and out must be device pointers");
    if (a->norm_type < KM_NORM_L1 || a->norm_type > KM_NORM_P)
        return fail(KM_ERR_BAD_ENUM, "norm_type %d is not a KmNormType", a->norm_type);
    if ((a->k > 1 && a->lda < a->m) || (a->n > 1 && a->ldb < a->k) || (a->o > 1 && a->ldc < a->k) ||
        (a->n > 1 && a->ldd < a->m) || (a->n > 1 && a->out_stride_n < a->m))
        return fail(KM_ERR_BAD_STRIDE, "a row pitch is smaller than the row it spans");
    if (a->a_stride_l < 0 || a->b_stride_l < 0 || a->c_stride_l < 0 || a->d_stride_l < 0 || a->out_stride_l < 0 ||
        a->out_stride_o < 0)
        return fail(KM_ERR_BAD_STRIDE, "strides must be non-negative");
    if (a->l > 1 && a->out_stride_l == 0) return fail(KM_ERR_BAD_STRIDE, "out cannot be broadcast over the batch");
    if (!hyper_ok(a->p)) return fail(KM_ERR_BAD_HYPERPARAM, "p needs a non-negative batch stride");
    if (a->split_k < 0) return fail(KM_ERR_BAD_SHAPE, "split_k must be >= 0");
    if (a->contraction < KM_CONTRACT_AUTO || a->contraction > KM_CONTRACT_TENSOR)
        return fail(KM_ERR_BAD_ENUM, "contraction must be KM_CONTRACT_AUTO, _FP32 or _TENSOR");

    GradParams& p = plan->p;
    p.M = a->m; p.N = a->n; p.O = a->o; p.K = a->k; p.L = a->l;
    p.A = a->a; p.lda = a->lda; p.a_sl = a->a_stride_l;
    p.B = a->b; p.ldb = a->ldb; p.b_sl = a->b_stride_l;
    p.C = a->c; p.ldc = a->ldc; p.c_sl = a->c_stride_l;
    p.D = a->d; p.ldd = a->ldd; p.d_sl = a->d_stride_l;
    p.p = a->p;
    int ot = 1;
    while (ot < a->o && ot < 16) ot *= 2;
    // The tensor-core kernel forms each weight once for up to 64 channels and leaves the channel
    // products to the MMA.  Up to 16 channels the FP32 kernel is level or faster (K = 30000, M = 4096,
    // N = 256: 20.4 against 19.1 ms at 16, 20.3 when the operands cannot be staged by TMA); from 17 on
    // it needs a second pass and the tensor cores win (40.4 against 22.0 ms at 32, 80.7 against 29.6 at
    // 64).  The tensor kernel needs at least one slab of k.
    plan->tensor = a->k > 0 && (a->contraction == KM_CONTRACT_TENSOR ||
                                (a->contraction == KM_CONTRACT_AUTO && a->o >= KM_GRAD_TENSOR_MIN_O && a->k >= 8 * G_BK));
    if (plan->tensor) ot = gt_ot_for(a->o);
    plan->ot = ot;
    plan->nt = nt_for(ot);
    p.tiles_m  = (int)ceil_div_ll(p.M, plan->tensor ? GT_TM : G_TM);
    p.tiles_n  = (int)ceil_div_ll(p.N, plan->tensor ? gt_tn_for(ot) : 16 * plan->nt);
    p.o_chunks = (int)ceil_div_ll(p.O > 0 ? p.O : 1, ot);
    p.a_vec    = aligned16(p.A) && p.lda % 4 == 0 && p.a_sl % 4 == 0;
    if ((long long)p.tiles_m * p.tiles_n > (1LL << 26)) return fail(KM_ERR_TOO_LARGE, "too many output tiles");
    if (p.o_chunks > 65535) return fail(KM_ERR_TOO_LARGE, "too many output channels");

    // Preferred k split.  Thread blocks run two per SM, in waves of `slots`; a launch of `blocks`
    // blocks takes ceil(blocks / slots) waves however full the last one is.  Among the splits the
    // k range allows (at least 8 slabs of k per block, at most 64 splits) take the smallest one
    // whose waves are within 2 % of the best filled; a launch that already fills its waves to 90 %
    // is left alone (every split costs a partial result written and read back).
    const long long blocks = (long long)p.tiles_m * p.tiles_n * p.o_chunks * p.L;
    const long long slots  = (long long)(plan->tensor ? gt_blocks_per_sm(plan->ot) : grad_min_blocks(plan->ot, plan->nt)) * sm_count();
    auto fill = [&](long long s) {
        const long long b = blocks * s;
        return (double)b / (double)(ceil_div_ll(b, slots) * slots);
    };
    int want = 1;
    if (blocks > 0 && fill(1) < 0.90) {
        int max_s = (int)(p.K / (8 * G_BK));
        if (max_s > 64) max_s = 64;
        double best = fill(1);
        for (int s = 2; s <= max_s; ++s) best = fill(s) > best ? fill(s) : best;
        for (int s = 1; s <= max_s; ++s)
            if (fill(s) >= best - 0.02) { want = s; break; }
    }
    plan->splits_wanted = want;
    plan->partial_elems = (long long)p.L * p.O * p.N * p.M;
    return 0;
}

}  // namespace
}  // namespace km

extern "C" int64_t kermac_b200_cdist_grad_scratch_bytes(const KmGradArgs* args) {
    using namespace km;
    GradPlan plan;
    if (make_grad_plan(args, &plan)) return 0;
    int splits = args->split_k > 0 ? args->split_k : plan.splits_wanted;
    if (splits <= 1) return 0;
    return (int64_t)splits * plan.partial_elems * 4;
}

extern "C" int kermac_b200_cdist_grad(const KmGradArgs* args, void* stream) {
    using namespace km;
    GradPlan plan;
    if (int rc = make_grad_plan(args, &plan)) return rc;
    GradParams& p = plan.p;
    if (p.M == 0 || p.N == 0 || p.O == 0) return 0;
    if (int rc = require_sm100()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    int splits = args->split_k > 0 ? args->split_k : plan.splits_wanted;
    if (splits > 1) {
        const int64_t need = (int64_t)splits * plan.partial_elems * 4;
        if (!args->scratch || args->scratch_bytes < need) {
            if (args->split_k > 1)
                return fail(KM_ERR_BAD_SHAPE, "split_k=%d needs %lld bytes of scratch, got %lld", splits, (long long)need,
                            (long long)(args->scratch ? args->scratch_bytes : 0));
            splits = 1;   // automatic mode falls back to a single pass
        }
    }
    int slabs       = (int)ceil_div_ll(p.K > 0 ? p.K : 1, G_BK);
    p.k_per_split   = (int)ceil_div_ll(slabs, splits) * G_BK;
    splits          = (int)ceil_div_ll(p.K > 0 ? p.K : 1, p.k_per_split);
    p.splits        = splits;
    if (splits > 1) {
        p.E = static_cast<float*>(args->scratch);
        p.e_sn = p.M; p.e_so = (long long)p.N * p.M; p.e_sl = (long long)p.O * p.N * p.M;
        p.split_stride = plan.partial_elems;
        p.e_vec = aligned16(p.E) && p.M % 4 == 0;
    } else {
        p.E = args->out;
        p.e_sn = args->out_stride_n; p.e_so = args->out_stride_o; p.e_sl = args->out_stride_l;
        p.split_stride = 0;
        p.e_vec = aligned16(p.E) && p.e_sn % 4 == 0 && p.e_so % 4 == 0 && p.e_sl % 4 == 0;
    }
    // a host scalar p = 1.5 means |x|^(1/2): the square-root kernels; a device vector of p is only
    // known to the kernel, which then takes the general lg2 / ex2 route
    const bool sqrt_route = (args->norm_type == KM_NORM_P && !args->p.ptr && args->p.value == 1.5f);
    if (plan.tensor) {
        GradTensorParams t;
        t.M = p.M; t.N = p.N; t.O = p.O; t.K = p.K; t.L = p.L;
        t.A = p.A; t.lda = p.lda; t.a_sl = p.a_sl;
        t.B = p.B; t.ldb = p.ldb; t.b_sl = p.b_sl;
        t.C = p.C; t.ldc = p.ldc; t.c_sl = p.c_sl;
        t.D = p.D; t.ldd = p.ldd; t.d_sl = p.d_sl;
        t.E = p.E; t.e_sn = p.e_sn; t.e_so = p.e_so; t.e_sl = p.e_sl;
        t.p = p.p;
        t.ot = plan.ot;
        t.rg = gt_rg_for(plan.ot);
        t.tiles_m = p.tiles_m; t.tiles_n = p.tiles_n; t.o_chunks = p.o_chunks; t.splits = p.splits;
        t.k_per_split = p.k_per_split; t.split_stride = p.split_stride;
        t.c_vec = aligned16(p.C) && p.ldc % 4 == 0 && p.c_sl % 4 == 0;
        if (int rc = grad_tensor_launch(t, sqrt_route ? GT_NORM_SQRT : args->norm_type, st)) return rc;
    } else {
    GradChoice choice = {nullptr, 0};
    switch (args->norm_type) {
        case KM_NORM_L1: choice = grad_fn_for<KM_NORM_L1>(plan.ot); break;
        case KM_NORM_L2: choice = grad_fn_for<KM_NORM_L2>(plan.ot); break;
        default: choice = sqrt_route ? grad_fn_for<G_NORM_SQRT>(plan.ot) : grad_fn_for<KM_NORM_P>(plan.ot); break;
    }
    GradFn fn = choice.fn;
    if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, choice.smem_bytes),
                             "cudaFuncSetAttribute(grad_kernel)"))
        return rc;
    dim3 grid((unsigned)((long long)p.tiles_m * p.tiles_n * splits), (unsigned)p.o_chunks, (unsigned)p.L);
    fn<<<grid, G_THREADS, choice.smem_bytes, st>>>(p);
    if (int rc = cuda_status(cudaGetLastError(), "launch of grad_kernel")) return rc;
    }
    if (splits > 1) {
        const long long total = plan.partial_elems;
        int blocks = (int)(ceil_div_ll(total, 256) < 4LL * sm_count() ? ceil_div_ll(total, 256) : 4LL * sm_count());
        grad_reduce_kernel<<<blocks, 256, 0, st>>>(p.E, args->out, p.M, p.N, p.O, p.L, splits, plan.partial_elems,
                                                   args->out_stride_n, args->out_stride_o, args->out_stride_l);
        if (int rc = cuda_status(cudaGetLastError(), "launch of grad_reduce_kernel")) return rc;
    }
    return 0;
}

// ---------------------------------------------------------------------------
// kermac_b200_cdist_grad_static: the split-k gradient for callers that have no way
// to hand over scratch memory.
//
// Some hosts of this library may not allocate device memory at the point where they
// call it: a plugin running inside another runtime's memory pool with a fixed budget,
// a real-time loop whose latency budget excludes allocator calls, or a binding whose
// foreign-function layer only passes through the pointers it was given.  For them the
// partial sums of the k split live in the array below, which is part of the library
// image: every GPU that loads the library carries it (KM_GRAD_STATIC_SCRATCH_BYTES)
// from load until the process exits.
//
// Rules that follow from sharing one array:
//   * it keeps whatever the previous call left in it.  Nothing in it has to start at
//     zero, because every partial tile a call reads back is first written in full by
//     that same call;
//   * two calls whose kernels overlap on the GPU (different streams, different host
//     threads) would write the same partials and corrupt each other: callers must
//     order them;
//   * the first call on each device looks up the array's device address.  That lookup
//     is a runtime API call, so make the first call per device outside any stream
//     capture.  The library calls no allocator, but the CUDA runtime places the array
//     when it loads this module on a device (at the latest during that first call), so
//     that warm-up call also belongs outside any region that must not see device memory
//     being reserved;
//   * the looked-up address is kept per device ordinal for the life of the process: it
//     does not survive cudaDeviceReset() or the teardown of the device's primary context.
namespace km {
namespace {

constexpr long long KM_GRAD_STATIC_FLOATS = KM_GRAD_STATIC_SCRATCH_BYTES / 4;
static __device__ __align__(256) float g_grad_static_scratch[KM_GRAD_STATIC_FLOATS];

// Device address of g_grad_static_scratch per device ordinal.  In host code the
// array's name only stands for the symbol; the address a kernel can use has to be
// asked for with the owning device current.
float*     g_grad_static_ptr[64] = {nullptr};
std::mutex g_grad_static_mutex;

int grad_static_scratch(float** out) {
    int dev = -1;
    if (int rc = cuda_status(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64) return fail(KM_ERR_INTERNAL, "device ordinal %d is out of range", dev);
    std::lock_guard<std::mutex> lock(g_grad_static_mutex);
    if (!g_grad_static_ptr[dev]) {
        void* p = nullptr;
        if (int rc = cuda_status(cudaGetSymbolAddress(&p, g_grad_static_scratch),
                                 "cudaGetSymbolAddress(g_grad_static_scratch)"))
            return rc;
        if (!p) return fail(KM_ERR_INTERNAL, "the static scratch array has no device address");
        g_grad_static_ptr[dev] = static_cast<float*>(p);
    }
    *out = g_grad_static_ptr[dev];
    return 0;
}

}  // namespace
}  // namespace km

extern "C" int kermac_b200_cdist_grad_static(const KmGradArgs* args, void* stream) {
    using namespace km;
    if (!args) return fail(KM_ERR_NULL_POINTER, "args is NULL");
    KmGradArgs local   = *args;
    local.scratch      = nullptr;
    local.scratch_bytes = 0;
    GradPlan plan;
    if (int rc = make_grad_plan(&local, &plan)) return rc;
    const int64_t cap      = KM_GRAD_STATIC_FLOATS * 4;
    const int64_t per_split = plan.partial_elems * 4;
    if (local.split_k > 1) {
        // an explicit split either fits the built-in array or is refused
        const int64_t need = (int64_t)local.split_k * per_split;
        if (need > cap)
            return fail(KM_ERR_TOO_LARGE,
                        "split_k = %d needs %lld bytes of scratch but the built-in array holds %lld; pass a smaller "
                        "split_k (1 always fits), or call kermac_b200_cdist_grad with your own scratch",
                        local.split_k, (long long)need, (long long)cap);
    } else if (local.split_k == 0) {
        // automatic: the preferred split, reduced to the largest one whose partial sums fit (down to a
        // single pass), as kermac_b200_cdist_grad does when the caller's scratch is too small
        long long fit = per_split > 0 ? cap / per_split : plan.splits_wanted;
        int splits    = plan.splits_wanted;
        if (splits > fit) splits = (int)fit;
        local.split_k = splits > 1 ? splits : 1;
    }
    if (local.split_k > 1) {
        float* ptr = nullptr;
        if (int rc = grad_static_scratch(&ptr)) return rc;
        local.scratch       = ptr;
        local.scratch_bytes = cap;
    }
    return kermac_b200_cdist_grad(&local, stream);
}
