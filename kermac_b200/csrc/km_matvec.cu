// kermac_b200_kernel_matvec: y[l, n, o] = sum_m Kmat[l, m, n] * c[l, o, m] where
// Kmat is the kernel matrix kermac_b200_build_kernel would produce, which is never
// written to global memory.
//
// A thread block owns 128 rows n and walks m in chunks of 128.  For each chunk it
// builds the 128 x 128 kernel-matrix tile exactly as the build kernel does (same
// staging, same packed 8 x 8 register blocks, same outer chain and epsilon mask),
// parks the tile in shared memory, and contracts it with the chunk's coefficients
// c[o, m] into per-thread accumulators y[n, o..] that live in registers for the
// whole walk.  The sum over m is therefore taken in a fixed order inside one block.
// With split_m > 1 the m range is divided over several blocks whose partial sums go
// to caller-provided scratch and are added in a fixed order by a second kernel.
//
// The reference has no such kernel: callers materialise run_kernel(...)
// (src/kermac/build_a_kernel.py:158-394) and multiply afterwards.
#include "km_build_cpasync.cuh"
#include "km_host.h"

namespace km {
namespace {

constexpr int MV_THREADS = 256;
constexpr int MV_TILE    = 128;
constexpr int MV_BK      = 16;
constexpr int MV_STAGES  = 2;
constexpr int MV_PITCH   = CPA_PITCH;
constexpr int MV_STAGE_FLOATS = 2 * MV_BK * MV_PITCH;
constexpr int MV_KT_PITCH     = MV_TILE + 4;   // kernel-matrix tile rows [n][m]

struct MatvecParams {
    int M, N, K, O, L;
    const float* A; long long a_sm, a_sk, a_sl;
    const float* B; long long b_sn, b_sk, b_sl;
    const float* C; long long ldc, c_sl;
    float*       Y; long long y_sn, y_so, y_sl;     // destination (y, or scratch when split)
    int inner_id, outer_power, kernel_type;
    KmHyper p_inner, p_outer, bandwidth;
    float epsilon;
    int tiles_n, splits, o_chunks;
    int m_per_split;                                  // multiple of MV_TILE
    long long split_stride;
};

template <int OT>
constexpr int mv_smem_bytes() {
    return (MV_STAGES * MV_STAGE_FLOATS + MV_TILE * MV_KT_PITCH + MV_TILE * OT) * 4;
}

template <int INNER, int OT, bool AVEC, bool BVEC>
__global__ void __launch_bounds__(MV_THREADS, 2) matvec_kernel(const __grid_constant__ MatvecParams p) {
    constexpr int OH = OT / 2;   // outputs per thread: one row n, OH channels
    extern __shared__ __align__(16) float smem[];
    float* s_kt = smem + MV_STAGES * MV_STAGE_FLOATS;     // [128 n][MV_KT_PITCH]
    float* s_c  = s_kt + MV_TILE * MV_KT_PITCH;           // [128 m][OT]

    const int tid  = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int tn    = blockIdx.x % p.tiles_n;
    const int split = blockIdx.x / p.tiles_n;
    const int oc    = blockIdx.y;
    const int l     = blockIdx.z;
    const int n0 = tn * MV_TILE;
    const int o0 = oc * OT;
    const int m_begin = split * p.m_per_split;
    const int m_end   = min(p.M, m_begin + p.m_per_split);
    const int chunks  = (m_end > m_begin) ? (m_end - m_begin + MV_TILE - 1) / MV_TILE : 0;

    const float* A = p.A + (long long)l * p.a_sl;
    const float* B = p.B + (long long)l * p.b_sl + (long long)n0 * p.b_sn;
    const float* C = p.C + (long long)l * p.c_sl;
    const int rem_n = p.N - n0;
    const int K = p.K;
    const int ktiles = K > 0 ? (K + MV_BK - 1) / MV_BK : 1;   // K = 0 still runs the outer chain on a zero sum
    const int total  = chunks * ktiles;

    const float p_inner = (INNER == IN_DIFF_POW || INNER == IN_DOT_POW) ? read_hyper(p.p_inner, l) : 0.0f;
    const Epilogue epi  = make_epilogue(p.outer_power, p.kernel_type, p.p_outer, p.bandwidth, p.epsilon, l);

    const int lm = lane & 7, ln = lane >> 3;
    const int wm = warp & 1, wn = warp >> 1;
    const int tm_off = wm * 64 + lm * 4;
    const int tn_off = wn * 32 + ln * 4;

    // contraction role of this thread
    const int cn = tid & (MV_TILE - 1);
    const int ch = tid >> 7;
    u64 yacc[OH / 2 > 0 ? OH / 2 : 1];
#pragma unroll
    for (int i = 0; i < (OH / 2 > 0 ? OH / 2 : 1); ++i) yacc[i] = 0ull;

    u64 acc[8][4];
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[j][i] = 0ull;

    auto stage = [&](int it) {
        const int chunk = it / ktiles, kt = it - chunk * ktiles;
        const int mc0   = m_begin + chunk * MV_TILE;
        float* st       = smem + (it % MV_STAGES) * MV_STAGE_FLOATS;
        stage_operand<AVEC, MV_BK>(st, A + (long long)mc0 * p.a_sm, p.a_sm, p.a_sk, m_end - mc0, K, kt, tid);
        stage_operand<BVEC, MV_BK>(st + MV_BK * MV_PITCH, B, p.b_sn, p.b_sk, rem_n, K, kt, tid);
    };

    if (total > 0) stage(0);
    cp_async_commit();

    for (int it = 0; it < total; ++it) {
        const int chunk = it / ktiles, kt = it - chunk * ktiles;
        cp_async_wait<0>();
        __syncthreads();
        if (it + 1 < total) stage(it + 1);
        cp_async_commit();

        const float* sa = smem + (it % MV_STAGES) * MV_STAGE_FLOATS + tm_off;
        const float* sb = smem + (it % MV_STAGES) * MV_STAGE_FLOATS + MV_BK * MV_PITCH + tn_off;
        consume_slab<INNER, MV_BK, MV_PITCH>(acc, sa, sb, K - kt * MV_BK, p_inner, 1.0f);

        if (kt == ktiles - 1) {
            const int mc0 = m_begin + chunk * MV_TILE;
            // kernel-matrix values of this chunk -> shared memory, [n][m]; columns of
            // m outside the range are zeroed so they add nothing.
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int nn = tn_off + (j >> 2) * 16 + (j & 3);
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int mm = tm_off + h * 32;
                    float v[4];
                    unpack2(acc[j][2 * h], v[0], v[1]);
                    unpack2(acc[j][2 * h + 1], v[2], v[3]);
#pragma unroll
                    for (int e = 0; e < 4; ++e) v[e] = (mc0 + mm + e < m_end) ? epi(v[e]) : 0.0f;
                    *reinterpret_cast<float4*>(s_kt + nn * MV_KT_PITCH + mm) = make_float4(v[0], v[1], v[2], v[3]);
                    acc[j][2 * h] = acc[j][2 * h + 1] = 0ull;
                }
            }
            // coefficients of this chunk -> shared memory, [m][o]
            for (int idx = tid; idx < MV_TILE * OT; idx += MV_THREADS) {
                const int mm = idx & (MV_TILE - 1), o = idx >> 7;
                const bool ok = (mc0 + mm < m_end) && (o0 + o < p.O);
                s_c[mm * OT + o] = ok ? C[(long long)(o0 + o) * p.ldc + mc0 + mm] : 0.0f;
            }
            __syncthreads();
            if constexpr (OT >= 4) {
#pragma unroll 2
                for (int mm = 0; mm < MV_TILE; mm += 4) {
                    const float4 k4  = *reinterpret_cast<const float4*>(s_kt + cn * MV_KT_PITCH + mm);
                    const float kv[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const u64 kd  = pack2(kv[e], kv[e]);
                        const u64* cp = reinterpret_cast<const u64*>(s_c + (mm + e) * OT + ch * OH);
#pragma unroll
                        for (int i = 0; i < OH / 2; ++i) yacc[i] = fma2(kd, cp[i], yacc[i]);
                    }
                }
            } else {
                // OT == 2: one channel per thread half
                float y0, y1;
                unpack2(yacc[0], y0, y1);
#pragma unroll 8
                for (int mm = 0; mm < MV_TILE; ++mm) y0 = fmaf(s_kt[cn * MV_KT_PITCH + mm], s_c[mm * OT + ch], y0);
                yacc[0] = pack2(y0, y1);
            }
            // the next chunk's epilogue overwrites s_kt / s_c only after the barrier at
            // the top of a later iteration, which every thread passes after this point
        }
    }
    cp_async_wait<0>();

    const int n = n0 + cn;
    if (n < p.N) {
        float* yrow = p.Y + (long long)split * p.split_stride + (long long)l * p.y_sl + (long long)n * p.y_sn;
        if constexpr (OT >= 4) {
#pragma unroll
            for (int i = 0; i < OH / 2; ++i) {
                float v0, v1;
                unpack2(yacc[i], v0, v1);
                const int o = o0 + ch * OH + 2 * i;
                if (o < p.O) yrow[(long long)o * p.y_so] = v0;
                if (o + 1 < p.O) yrow[(long long)(o + 1) * p.y_so] = v1;
            }
        } else {
            float v0, v1;
            unpack2(yacc[0], v0, v1);
            const int o = o0 + ch;
            if (o < p.O) yrow[(long long)o * p.y_so] = v0;
        }
    }
}

__global__ void __launch_bounds__(256) matvec_reduce_kernel(const float* __restrict__ partial, float* __restrict__ y,
                                                            int N, int O, int L, int splits, long long split_stride,
                                                            long long y_sn, long long y_so, long long y_sl) {
    const long long total = (long long)L * N * O;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        float s = 0.0f;
        for (int sp = 0; sp < splits; ++sp) s += partial[sp * split_stride + i];
        long long r = i;
        const int o = (int)(r % O); r /= O;
        const int n = (int)(r % N); r /= N;
        const int l = (int)r;
        y[l * y_sl + n * y_sn + o * y_so] = s;
    }
}

typedef void (*MatvecFn)(const MatvecParams);

template <int INNER, int OT>
MatvecFn mv_pick_layout(bool avec, bool bvec) {
    if (avec && bvec) return matvec_kernel<INNER, OT, true, true>;
    if (avec) return matvec_kernel<INNER, OT, true, false>;
    if (bvec) return matvec_kernel<INNER, OT, false, true>;
    return matvec_kernel<INNER, OT, false, false>;
}
template <int INNER>
MatvecFn mv_pick_ot(int ot, bool avec, bool bvec) {
    switch (ot) {
        case 2: return mv_pick_layout<INNER, 2>(avec, bvec);
        case 4: return mv_pick_layout<INNER, 4>(avec, bvec);
        case 8: return mv_pick_layout<INNER, 8>(avec, bvec);
        default: return mv_pick_layout<INNER, 16>(avec, bvec);
    }
}
MatvecFn mv_pick(int inner, int ot, bool avec, bool bvec) {
    switch (inner) {
        case IN_DIFF_ABS: return mv_pick_ot<IN_DIFF_ABS>(ot, avec, bvec);
        case IN_DIFF_SQUARE: return mv_pick_ot<IN_DIFF_SQUARE>(ot, avec, bvec);
        case IN_DIFF_POW: return mv_pick_ot<IN_DIFF_POW>(ot, avec, bvec);
        case IN_DOT_NOOP: return mv_pick_ot<IN_DOT_NOOP>(ot, avec, bvec);
    }
    return nullptr;
}
int mv_smem_for(int ot) {
    switch (ot) {
        case 2: return mv_smem_bytes<2>();
        case 4: return mv_smem_bytes<4>();
        case 8: return mv_smem_bytes<8>();
        default: return mv_smem_bytes<16>();
    }
}

bool mv_layout_ok(long long rows, long long cols, long long s_row, long long s_col) {
    if (rows <= 0 || cols <= 0) return true;
    return (s_col == 1 && s_row >= cols) || (s_row == 1 && s_col >= rows);
}

struct MatvecPlan {
    MatvecParams p;
    int ot;
    bool avec, bvec;
    int splits_wanted;
    long long partial_elems;
};

int make_matvec_plan(const KmMatvecArgs* a, MatvecPlan* plan) {
    if (!a) return fail(KM_ERR_NULL_POINTER, "args is NULL");
    if (a->m < 0 || a->n < 0 || a->k < 0 || a->o < 0 || a->l < 1)
        return fail(KM_ERR_BAD_SHAPE, "bad extents m=%d n=%d k=%d o=%d l=%d", a->m, a->n, a->k, a->o, a->l);
    if (a->l > 65535) return fail(KM_ERR_TOO_LARGE, "at most 65535 batch entries per call");
    const bool empty = (a->n == 0 || a->o == 0);
    if (!empty && (!a->y || (a->m > 0 && (!a->c || (a->k > 0 && (!a->a || !a->b))))))
        return fail(KM_ERR_NULL_POINTER, "a, b, c and y must be device pointers");
    if (a->inner_operator < 0 || a->inner_operator > KM_INNER_DOT || a->inner_power < 0 || a->inner_power > KM_POW_POW ||
        a->outer_power < 0 || a->outer_power > KM_POW_POW || a->kernel_type < 0 || a->kernel_type > KM_KERNEL_GAUSSIAN)
        return fail(KM_ERR_BAD_ENUM, "descriptor enums out of range");
    if (!mv_layout_ok(a->m, a->k, a->a_stride_m, a->a_stride_k))
        return fail(KM_ERR_BAD_STRIDE, "a has a non-standard memory layout");
    if (!mv_layout_ok(a->n, a->k, a->b_stride_n, a->b_stride_k))
        return fail(KM_ERR_BAD_STRIDE, "b has a non-standard memory layout");
    if (a->o > 1 && a->ldc < a->m) return fail(KM_ERR_BAD_STRIDE, "ldc is smaller than m");
    if (a->a_stride_l < 0 || a->b_stride_l < 0 || a->c_stride_l < 0 || a->y_stride_l < 0 || a->y_stride_n < 0 ||
        a->y_stride_o < 0)
        return fail(KM_ERR_BAD_STRIDE, "strides must be non-negative");
    if (!hyper_ok(a->p_inner) || !hyper_ok(a->p_outer) || !hyper_ok(a->bandwidth))
        return fail(KM_ERR_BAD_HYPERPARAM, "hyper-parameter vectors need a non-negative batch stride");
    if (a->split_m < 0) return fail(KM_ERR_BAD_SHAPE, "split_m must be >= 0");

    MatvecParams& p = plan->p;
    p.M = a->m; p.N = a->n; p.K = a->k; p.O = a->o; p.L = a->l;
    p.A = a->a; p.a_sm = a->a_stride_m; p.a_sk = a->a_stride_k; p.a_sl = a->a_stride_l;
    p.B = a->b; p.b_sn = a->b_stride_n; p.b_sk = a->b_stride_k; p.b_sl = a->b_stride_l;
    p.C = a->c; p.ldc = a->ldc; p.c_sl = a->c_stride_l;
    p.inner_id = inner_id(a->inner_operator, a->inner_power);
    if (!mv_pick(p.inner_id, 16, false, false))
        return fail(KM_ERR_BAD_ENUM, "kernel_matvec supports the inner steps |b-a|, (b-a)^2, |b-a|^p and b*a");
    p.outer_power = a->outer_power;
    p.kernel_type = a->kernel_type;
    p.p_inner = a->p_inner; p.p_outer = a->p_outer; p.bandwidth = a->bandwidth;
    p.epsilon = a->epsilon;
    int ot = 2;
    while (ot < a->o && ot < 16) ot *= 2;
    plan->ot   = ot;
    p.tiles_n  = (int)ceil_div_ll(p.N, MV_TILE);
    p.o_chunks = (int)ceil_div_ll(p.O > 0 ? p.O : 1, ot);
    if (p.o_chunks > 65535) return fail(KM_ERR_TOO_LARGE, "too many output channels");
    plan->avec = (p.a_sm == 1) && aligned16(p.A) && (p.a_sk % 4 == 0 || p.K <= 1) && (p.a_sl % 4 == 0);
    plan->bvec = (p.b_sn == 1) && aligned16(p.B) && (p.b_sk % 4 == 0 || p.K <= 1) && (p.b_sl % 4 == 0);

    // Preferred m split: fill whole waves of 2 blocks per SM when the row tiles alone
    // leave more than ~10 % of a wave idle.
    const long long blocks = (long long)p.tiles_n * p.o_chunks * p.L;
    const long long slots  = 2LL * sm_count();
    int want = 1;
    if (blocks > 0) {
        const double waves = (double)blocks / (double)slots;
        const double eff   = waves / (double)ceil_div_ll(blocks, slots);
        if (eff < 0.9) {
            // smallest split that brings the efficiency above 0.95, capped by chunk count
            const int max_split = (int)ceil_div_ll(p.M > 0 ? p.M : 1, 8 * MV_TILE);
            for (int s = 2; s <= 32 && s <= max_split; ++s) {
                const double w = (double)(blocks * s) / (double)slots;
                if (w / (double)ceil_div_ll(blocks * s, slots) >= 0.95) { want = s; break; }
                want = s;
            }
        }
    }
    plan->splits_wanted = want;
    plan->partial_elems = (long long)p.L * p.N * p.O;
    return 0;
}

}  // namespace
}  // namespace km

extern "C" int64_t kermac_b200_kernel_matvec_scratch_bytes(const KmMatvecArgs* args) {
    using namespace km;
    MatvecPlan plan;
    if (make_matvec_plan(args, &plan)) return 0;
    int splits = args->split_m > 0 ? args->split_m : plan.splits_wanted;
    if (splits <= 1) return 0;
    return (int64_t)splits * plan.partial_elems * 4;
}

extern "C" int kermac_b200_kernel_matvec(const KmMatvecArgs* args, void* stream) {
    using namespace km;
    MatvecPlan plan;
    if (int rc = make_matvec_plan(args, &plan)) return rc;
    MatvecParams& p = plan.p;
    if (p.N == 0 || p.O == 0) return 0;
    if (int rc = require_sm100()) return rc;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    int splits = args->split_m > 0 ? args->split_m : plan.splits_wanted;
    if (splits > 1) {
        const int64_t need = (int64_t)splits * plan.partial_elems * 4;
        if (!args->scratch || args->scratch_bytes < need) {
            if (args->split_m > 1)
                return fail(KM_ERR_BAD_SHAPE, "split_m=%d needs %lld bytes of scratch, got %lld", splits, (long long)need,
                            (long long)(args->scratch ? args->scratch_bytes : 0));
            splits = 1;
        }
    }
    const int chunks = (int)ceil_div_ll(p.M > 0 ? p.M : 1, MV_TILE);
    p.m_per_split    = (int)ceil_div_ll(chunks, splits) * MV_TILE;
    splits           = (int)ceil_div_ll(p.M > 0 ? p.M : 1, p.m_per_split);
    p.splits         = splits;
    if (splits > 1) {
        p.Y = static_cast<float*>(args->scratch);
        p.y_so = 1; p.y_sn = p.O; p.y_sl = (long long)p.N * p.O;
        p.split_stride = plan.partial_elems;
    } else {
        p.Y = args->y;
        p.y_sn = args->y_stride_n; p.y_so = args->y_stride_o; p.y_sl = args->y_stride_l;
        p.split_stride = 0;
    }
    MatvecFn fn = mv_pick(p.inner_id, plan.ot, plan.avec, plan.bvec);
    if (!fn) return fail(KM_ERR_INTERNAL, "no matvec kernel for inner id %d", p.inner_id);
    const int smem_bytes = mv_smem_for(plan.ot);
    if (int rc = cuda_status(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes),
                             "cudaFuncSetAttribute(matvec_kernel)"))
        return rc;
    dim3 grid((unsigned)((long long)p.tiles_n * splits), (unsigned)p.o_chunks, (unsigned)p.L);
    fn<<<grid, MV_THREADS, smem_bytes, st>>>(p);
    if (int rc = cuda_status(cudaGetLastError(), "launch of matvec_kernel")) return rc;
    if (splits > 1) {
        const long long total = plan.partial_elems;
        int blocks = (int)(ceil_div_ll(total, 256) < 4LL * sm_count() ? ceil_div_ll(total, 256) : 4LL * sm_count());
        matvec_reduce_kernel<<<blocks, 256, 0, st>>>(p.Y, args->y, p.N, p.O, p.L, splits, plan.partial_elems,
                                                     args->y_stride_n, args->y_stride_o, args->y_stride_l);
        if (int rc = cuda_status(cudaGetLastError(), "launch of matvec_reduce_kernel")) return rc;
    }
    return 0;
}
