// Kernel-matrix build, cp.async staged: handles every operand layout the host API
// accepts (either majorness, any pitch, any base alignment).
//
// A thread block of 256 threads owns one 128 (m) x 128 (n) output tile and walks
// k in slabs of 32 through a 3-stage cp.async pipeline.  Both operands are staged
// k-major with the tile dimension contiguous ([k][128 + pad]) whatever their
// layout in global memory, so the math loop reads them with 128-bit shared loads:
//   - an operand whose tile dimension is contiguous and 16-byte aligned is copied
//     with 16-byte cp.async (edge chunks copy only their valid bytes, rest zero);
//   - any other operand is copied element-wise with 4-byte cp.async, walking
//     global memory along whichever stride is 1.
// Each thread accumulates an 8 x 8 block as packed pairs (see inner_block).
//
// Computes what the reference's kernel_cute_build_kernel computes
// (include/build_a_kernel.cuh:19-463); staging, thread mapping and instruction
// selection are new.
#pragma once

#include "km_build_params.cuh"

namespace km {

constexpr int CPA_TILE    = BUILD_TILE;
constexpr int CPA_BK      = BUILD_CPA_BK;
constexpr int CPA_STAGES  = BUILD_CPA_STAGES;
constexpr int CPA_PITCH   = BUILD_CPA_PITCH;
constexpr int CPA_THREADS = BUILD_CPA_THREADS;
constexpr int CPA_STAGE_FLOATS = 2 * CPA_BK * CPA_PITCH;
constexpr int CPA_SMEM_BYTES   = BUILD_CPA_SMEM_BYTES;

// Stages the k slab `kt` (BK rows) of one operand tile into `dst` ([BK][CPA_PITCH]).
//   base  : first element of the tile (row 0 of the tile dimension, k = 0)
//   s_t   : stride of the tile dimension, s_k: stride of k
//   rem_t : valid extent of the tile dimension (may exceed 128)
template <bool VEC, int BK = CPA_BK>
__device__ __forceinline__ void stage_operand(float* dst, const float* base, long long s_t, long long s_k, int rem_t,
                                              int K, int kt, int tid) {
    const int k0 = kt * BK;
    if constexpr (VEC) {
#pragma unroll
        for (int i = 0; i < (BK * CPA_TILE / 4) / CPA_THREADS; ++i) {
            const int idx = tid + i * CPA_THREADS;
            const int kk  = idx >> 5;
            const int t   = (idx & 31) << 2;
            const int gk  = k0 + kk;
            int valid     = min(4, rem_t - t);
            valid         = (gk < K && valid > 0) ? valid : 0;
            const float* src = valid ? base + static_cast<long long>(gk) * s_k + t : base;
            cp_async_16(smem_u32(dst + kk * CPA_PITCH + t), src, valid * 4);
        }
    } else {
        const bool k_contig = (s_k == 1);
#pragma unroll
        for (int i = 0; i < (BK * CPA_TILE) / CPA_THREADS; ++i) {
            const int idx = tid + i * CPA_THREADS;
            int kk, t;
            if (k_contig) {
                kk = idx & (BK - 1);
                t  = idx / BK;
            } else {
                t  = idx & (CPA_TILE - 1);
                kk = idx >> 7;
            }
            const int  gk = k0 + kk;
            const bool ok = (gk < K) && (t < rem_t);
            const float* src = ok ? base + static_cast<long long>(t) * s_t + static_cast<long long>(gk) * s_k : base;
            cp_async_4(smem_u32(dst + kk * CPA_PITCH + t), src, ok ? 4 : 0);
        }
    }
}

// Applies the outer chain to one thread's 8 x 8 block and stores it.
// Coordinates: acc[j][mp] holds rows n = n_base + (j / 4) * 16 + (j % 4) and
// columns m = m_base + (mp / 2) * 32 + (mp % 2) * 2 + {0, 1}.
// With `mirror` the block is also written transposed, to C[m][n]: the kernel matrix of
// a symmetric problem, of which only the tiles on and above the diagonal are computed.
// MIRROR = false compiles the transposed stores out, so kernels of ordinary problems carry none of it.
template <int INNER, bool MIRROR>
__device__ __forceinline__ void finish_block(const BuildParams& p, int l, u64 (&acc)[8][4], int m_base, int n_base,
                                             bool mirror) {
    const Epilogue epi = make_epilogue(p.outer_power, p.kernel_type, p.p_outer, p.bandwidth, p.epsilon, l);
    float reg = 0.0f;
    if (p.kernel_type != KM_KERNEL_NONE) reg = read_hyper(p.regularization, l);
    float* C = p.C + static_cast<long long>(l) * p.c_sl;
    const bool mc = p.c_multicast != 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int n = n_base + (j >> 2) * 16 + (j & 3);
        if constexpr (!MIRROR) {
            if (n >= p.N) continue;
        }
        float* row = C + static_cast<long long>(n) * p.c_ld;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = m_base + h * 32;
            float v[4];
            unpack2(acc[j][2 * h], v[0], v[1]);
            unpack2(acc[j][2 * h + 1], v[2], v[3]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float x = v[e];
                if constexpr (INNER == IN_DIFF_NOOP) x *= p.sgn;
                x = epi(x);
                if (reg != 0.0f && (p.reg_off_m + m + e == p.reg_off_n + n)) x = 1.0f + reg;
                v[e] = x;
            }
            if constexpr (MIRROR) {
                acc[j][2 * h]     = pack2(v[0], v[1]);     // kept for the mirror image
                acc[j][2 * h + 1] = pack2(v[2], v[3]);
            }
            if (n >= p.N) continue;
            if (p.c_vec4 && m + 3 < p.M) {
                store_result4(row + m, v[0], v[1], v[2], v[3], mc);
            } else {
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    if (m + e < p.M) store_result1(row + m + e, v[e], mc);
            }
        }
    }
    if constexpr (!MIRROR) return;
    if (!mirror) return;
    // C[m][n]: for each of the thread's 8 columns m, its rows n come in two runs of four
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int m = m_base + (i >> 1) * 32 + (i & 1) * 2 + half;
            if (m >= p.M) continue;
            float* row = C + static_cast<long long>(m) * p.c_ld;
#pragma unroll
            for (int g = 0; g < 2; ++g) {
                const int n = n_base + g * 16;
                float v[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    float lo, hi;
                    unpack2(acc[g * 4 + e][i], lo, hi);
                    v[e] = half ? hi : lo;
                }
                if (p.c_vec4 && n + 3 < p.N) {
                    store_result4(row + n, v[0], v[1], v[2], v[3], mc);
                } else {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        if (n + e < p.N) store_result1(row + n + e, v[e], mc);
                }
            }
        }
    }
}

// SYM: a and b are the same matrix and the chain is symmetric in (m, n); see BuildParams::symmetric.
template <int INNER, bool AVEC, bool BVEC, bool SYM>
__global__ void __launch_bounds__(CPA_THREADS, 2) build_cpasync_kernel(const __grid_constant__ BuildParams p) {
    extern __shared__ __align__(16) float smem[];
    const int tid  = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int l    = blockIdx.y;

    int tm, tn;
    tile_coords(p.tile_first + blockIdx.x, p.tiles_m, p.tiles_n, p.panel, tm, tn);
    if (SYM && tn < tm) return;   // the tile's mirror image (tn, tm) writes this part of C
    const int m0 = tm * CPA_TILE;
    const int n0 = tn * CPA_TILE;

    const float* A = p.A + static_cast<long long>(l) * p.a_sl + static_cast<long long>(m0) * p.a_sm;
    const float* B = p.B + static_cast<long long>(l) * p.b_sl + static_cast<long long>(n0) * p.b_sn;
    const int rem_m = p.M - m0;
    const int rem_n = p.N - n0;
    const int K     = p.K;
    const int ktiles = (K + CPA_BK - 1) / CPA_BK;

    const float p_inner = (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) ? read_hyper(p.p_inner, l) : 0.0f;

    // thread -> sub-block of the tile
    const int lm = lane & 7, ln = lane >> 3;
    const int wm = warp & 1, wn = warp >> 1;
    const int tm_off = wm * 64 + lm * 4;   // + {0, 32}
    const int tn_off = wn * 32 + ln * 4;   // + {0, 16}

    u64 acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0ull;

#pragma unroll
    for (int s = 0; s < CPA_STAGES - 1; ++s) {
        if (s < ktiles) {
            float* st = smem + s * CPA_STAGE_FLOATS;
            stage_operand<AVEC>(st, A, p.a_sm, p.a_sk, rem_m, K, s, tid);
            stage_operand<BVEC>(st + CPA_BK * CPA_PITCH, B, p.b_sn, p.b_sk, rem_n, K, s, tid);
        }
        cp_async_commit();
    }

    for (int kt = 0; kt < ktiles; ++kt) {
        cp_async_wait<CPA_STAGES - 2>();
        __syncthreads();
        {
            const int nk = kt + CPA_STAGES - 1;
            if (nk < ktiles) {
                float* st = smem + (nk % CPA_STAGES) * CPA_STAGE_FLOATS;
                stage_operand<AVEC>(st, A, p.a_sm, p.a_sk, rem_m, K, nk, tid);
                stage_operand<BVEC>(st + CPA_BK * CPA_PITCH, B, p.b_sn, p.b_sk, rem_n, K, nk, tid);
            }
            cp_async_commit();
        }
        const float* sa = smem + (kt % CPA_STAGES) * CPA_STAGE_FLOATS + tm_off;
        const float* sb = smem + (kt % CPA_STAGES) * CPA_STAGE_FLOATS + CPA_BK * CPA_PITCH + tn_off;
        consume_slab<INNER, CPA_BK, CPA_PITCH>(acc, sa, sb, K - kt * CPA_BK, p_inner, p.sgn);
    }
    cp_async_wait<0>();

    finish_block<INNER, SYM>(p, l, acc, m0 + tm_off, n0 + tn_off, SYM && tm != tn);
}

}  // namespace km
